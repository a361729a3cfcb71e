"""Regenerate the golden fixtures in this directory from the unmodified reference.

Run in a container that has the reference checkout (no GPU needed):

    python tests/golden/make_golden.py --reference /path/to/reference

It imports the reference's own `trainkernel.capture` and
`trainkernel.reference.run`, drives them over this repository's seeded
workloads, and stores per case: the captured program (JSON), the loss of every
step, and samples plus float64 checksums of the last step's gradients and of the
final state.  The fixtures are what `tests/test_oracle_golden.py` pins
`oracle/interpreter.py` and the front end against; the reference itself is not
needed to run the tests.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from trainkernel_b200 import workloads  # noqa: E402

SAMPLE = 2048

# (case name, workload, seed, steps)
CASES = [
    ("c1_seed0", "c1", 0, 100),
    ("c2_seed0", "c2", 0, 100),
    ("c2_seed1", "c2", 1, 100),
    ("c2_seed2", "c2", 2, 100),
    ("c3_seed0", "c3", 0, 100),
    ("c3_seed1", "c3", 1, 100),
    ("c3_seed2", "c3", 2, 100),
    ("c4_seed0", "c4", 0, 100),
    ("gemv_seed0", "gemv", 0, 100),
]


def program_to_json(program) -> dict:
    def spec(s):
        return dataclasses.asdict(s)

    def operand(x):
        return spec(x) if dataclasses.is_dataclass(x) else {"scalar": x}

    return {
        "inputs": [spec(s) for s in program.inputs],
        "operations": [
            {"name": op.name, "op": op.op, "inputs": [operand(x) for x in op.inputs], "output": spec(op.output),
             "attrs": {k: (list(v) if isinstance(v, tuple) else v) for k, v in op.attrs.items()}}
            for op in program.operations
        ],
        "outputs": [spec(s) for s in program.outputs],
    }


def sample(t: torch.Tensor) -> np.ndarray:
    flat = t.detach().float().reshape(-1)
    stride = max(1, flat.numel() // SAMPLE)
    return flat[::stride][:SAMPLE].numpy().copy()


def checksum(t: torch.Tensor) -> np.ndarray:
    d = t.detach().double()
    return np.array([float(d.sum()), float(d.abs().sum())])


def leaves(state):
    return tuple(state) if isinstance(state, (tuple, list)) else (state,)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the unmodified reference project (arpjw/trainkernel)")
    parser.add_argument("--only", default=None)
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    import trainkernel as ref
    from trainkernel.reference import run as ref_run

    torch.backends.cuda.matmul.allow_tf32 = False
    programs = {}
    for case, name, seed, steps in CASES:
        if args.only and args.only != case:
            continue
        work = workloads.build(name, seed=seed)
        fn = work.fn()
        state = leaves(work.state)
        single = not isinstance(work.state, (tuple, list))
        n = len(state)
        x0, t0 = work.batches[0]
        program, _ = ref.capture(fn, (work.state, x0, t0))
        programs[case] = program_to_json(program)
        losses, eager_losses = [], []
        eager_state = work.state
        out = None
        for i in range(steps):
            x, t = work.batches[i % len(work.batches)]
            out = ref_run(program, (*state, x, t))
            losses.append(float(out[0]))
            state = tuple(o.clone() for o in out[1 + n:])
            if steps <= 100 and name != "c4":
                eager = fn(eager_state, x, t)
                eager_losses.append(float(eager[0]))
                eager_state = eager[2]
        record = {
            "losses": np.array(losses, dtype=np.float32),
            "eager_losses": np.array(eager_losses, dtype=np.float32),
            "input_checksum": np.stack([checksum(v) for v in (*leaves(work.state), x0, t0)]),
        }
        for i in range(n):
            record[f"grad{i}_sample"] = sample(out[1 + i])
            record[f"grad{i}_checksum"] = checksum(out[1 + i])
            record[f"state{i}_sample"] = sample(state[i])
            record[f"state{i}_checksum"] = checksum(state[i])
        np.savez_compressed(HERE / f"{case}.npz", **record)
        print(case, "ops", len(program.operations), "loss", losses[0], "->", losses[-1], "single" if single else n)

    # The reference's own irregular test shape (reference: tests/test_ir_reference.py:23-33),
    # in every supported dtype, three steps of the native-dtype MLP step.
    from benchmarks.train_mlp import make_inputs, step
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        params, x, target = make_inputs(7, 11, 17, 5, dtype, "cpu")
        fn = lambda p, xx, yy: step(p, xx, yy, 1e-3)  # noqa: E731
        program, _ = ref.capture(fn, (params, x, target))
        case = f"mlp_7_11_17_5_{str(dtype).split('.')[-1]}"
        programs[case] = program_to_json(program)
        record = {"input_checksum": np.stack([checksum(v) for v in (*params, x, target)])}
        record.update({f"param{i}": p.float().numpy() for i, p in enumerate(params)})
        record["x"], record["target"] = x.float().numpy(), target.float().numpy()
        state = params
        for s in range(3):
            out = ref_run(program, (*state, x, target))
            for j, o in enumerate(out):
                record[f"step{s}_out{j}"] = o.float().numpy()
            state = tuple(out[-4:])
        np.savez_compressed(HERE / f"{case}.npz", **record)
        print(case, "ops", len(program.operations))
    if not args.only:
        (HERE / "programs.json").write_text(json.dumps(programs, indent=0, sort_keys=True))


if __name__ == "__main__":
    main()
