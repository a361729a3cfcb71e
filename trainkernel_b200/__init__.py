"""B200-native (sm_100a) back end for TrainKernel-style compiled training steps.

Same public names as the reference package (reference: trainkernel/__init__.py:1-23).
"""
from .ir import Operation, Program, TensorSpec
from .frontend import (
    CapturedProgram,
    CompiledFunction,
    CompiledTrainingStep,
    capture,
    compile,
    compile_training,
)

__version__ = "0.1.0"

__all__ = [
    "TensorSpec",
    "Operation",
    "Program",
    "CapturedProgram",
    "CompiledFunction",
    "CompiledTrainingStep",
    "capture",
    "compile",
    "compile_training",
]
