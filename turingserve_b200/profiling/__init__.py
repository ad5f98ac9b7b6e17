"""Small single-kernel workloads for profiler captures (``python -m turingserve_b200.profiling``)."""
