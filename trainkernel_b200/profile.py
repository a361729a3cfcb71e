"""Per-stage timing of a compiled step from stamps written inside the kernel.

The reference measures stages by string-patching `%globaltimer` reads into the
generated source after every grid barrier (reference: scripts/profile_stages.py:36-54).
Here the generator emits those stamps itself when asked (`stage_stamps=True`)
and the runtime shim reads them back, so profiling is an option of `compile`,
not a source rewrite.
"""
from __future__ import annotations

from typing import Any, Callable, Sequence

import torch

from .frontend import compile, compile_training


def stage_profile(fn: Callable[..., Any], example_inputs: Sequence[Any], *, training: bool = True,
                  repeats: int = 10, **options: Any) -> list[dict]:
    """Compile `fn` with stage stamps, run it `repeats` times, and return one record per stage.

    Each record holds the stage index, the fastest and median duration in microseconds (a stage's
    time includes the grid barrier that ends it, as seen by block 0), and the units scheduled in it.
    State tensors in `example_inputs` are updated by the runs when `training` is true.
    """
    builder = compile_training if training else compile
    compiled = builder(fn, example_inputs, stage_stamps=True, **options)
    runner = compiled.runner
    for _ in range(3):
        compiled(*example_inputs)
    torch.cuda.synchronize(runner.device)
    samples: list[list[float]] = []
    for _ in range(repeats):
        compiled(*example_inputs)
        stamps = runner.stage_stamps()
        samples.append([(b - a) / 1e3 for a, b in zip(stamps[:-1], stamps[1:])])
    records = []
    for stage in range(runner.generated.stages):
        column = sorted(sample[stage] for sample in samples)
        units = [f"{name}:{kind}{'/' + path if path else ''}" for s, kind, name, path, _ in runner.generated.units if s == stage]
        records.append({"stage": stage, "min_us": column[0], "median_us": column[len(column) // 2], "units": units})
    return records
