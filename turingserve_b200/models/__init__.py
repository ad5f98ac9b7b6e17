"""Architectures: each module turns one family's config.json into a ModelConfig and registers it."""
