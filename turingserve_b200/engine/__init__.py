"""Step function, scheduler, engine loop and trace replay."""

from turingserve_b200.engine.batch import StepEntry, StepInputs
from turingserve_b200.engine.engine import FinalOutput, LLMEngine
from turingserve_b200.engine.request import Request, RequestOutput
from turingserve_b200.engine.runner import ModelRunner, run_needs
from turingserve_b200.engine.scheduler import Scheduler

__all__ = ["StepEntry", "StepInputs", "FinalOutput", "LLMEngine", "Request", "RequestOutput",
           "ModelRunner", "run_needs", "Scheduler"]
