"""Captured training-loop comparison: the compiled step against eager PyTorch, both under CUDA graphs.

Follows the protocol of the reference harness (reference: benchmarks/train_loop.py:90-161,
196-384): FP32 master weights and BF16 compute on a 2-layer MLP (or a one-hot classification
head), a correctness gate first (a 100-step trajectory and a captured replay, every loss, gradient
and update compared with eager PyTorch), then an N-step CUDA graph with state feedback per method,
timed in interleaved pairs with the state reset outside the timed replay.  Reported per method:
median / p10 / p90 per step, compile seconds cold and warm, capture seconds, kernel facts, speed
ratios with a bootstrap confidence interval, and the number of steps after which the set-up cost
is repaid.  The reference's Inductor arms are not part of this back end; the methods are

    megakernel     the compiled step returning fresh state tensors (state copied back by the loop)
    mega_inplace   the compiled step committing the update into the state tensors (compile_training)
    eager_graph    the eager PyTorch step

Run: `python -m trainkernel_b200.benchmarks.train_loop --batch 128 --input 512 --hidden 1024 --output 256`.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
from pathlib import Path
from typing import Callable, Sequence

import torch

from .. import compile as tk_compile
from .. import compile_training
from ..workloads import mlp_master_step

LR = 1e-3
# The reference's gates (reference: benchmarks/train_loop.py:73-87): FP32 loss and updates, BF16-computed gradients.
TOLERANCES = {"loss": (2e-4, 2e-5), "gradients": (0.04, 0.004), "updates": (2e-4, 2e-5)}


def make_problem(batch: int, input_size: int, hidden: int, output: int, device, batches: int, seed: int, task: str):
    """Seeded FP32 masters (values representable in BF16) and BF16 batches; a teacher provides the targets."""
    gen = torch.Generator(device="cpu").manual_seed(seed)

    def normal(shape, scale=1.0):
        return (torch.randn(shape, generator=gen) * scale).to(torch.bfloat16)

    sizes = ((input_size, hidden), (hidden, output))
    params, teacher = [], []
    for store in (params, teacher):
        for fan_in, fan_out in sizes:
            store.append(normal((fan_in, fan_out), fan_in ** -0.5))
            store.append(torch.zeros(fan_out, dtype=torch.bfloat16))
    data = []
    for _ in range(batches):
        x = normal((batch, input_size))
        with torch.no_grad():
            y = torch.relu(x.float() @ teacher[0].float() + teacher[1].float()) @ teacher[2].float() + teacher[3].float()
        if task == "classification-head":
            y = torch.nn.functional.one_hot(y.argmax(dim=1), output).float()
        data.append((x.to(device), y.to(torch.bfloat16).to(device)))
    return tuple(p.float().to(device) for p in params), data


def eager_step(params, x, target):
    return mlp_master_step(params, x, target, LR)


def check_step(actual, expected) -> dict[str, float]:
    """Compare (loss, grads, updated) triples under the gates; returns the largest absolute errors."""
    worst = {}
    groups = {"loss": ([actual[0]], [expected[0]]), "gradients": (actual[1], expected[1]), "updates": (actual[2], expected[2])}
    for kind, (got, want) in groups.items():
        rtol, atol = TOLERANCES[kind]
        worst[kind] = 0.0
        for a, b in zip(got, want):
            torch.testing.assert_close(a.float(), b.float(), rtol=rtol, atol=atol, msg=lambda m, kind=kind: f"{kind}: {m}")
            worst[kind] = max(worst[kind], float((a.float() - b.float()).abs().max()))
    return worst


def feed_back(state: Sequence[torch.Tensor], updated: Sequence[torch.Tensor]) -> None:
    for dst, src in zip(state, updated):
        if dst.data_ptr() != src.data_ptr():
            dst.copy_(src)


def trajectory(method: Callable, initial, batches, steps: int) -> dict:
    """Run `method` and eager PyTorch side by side from the same state, each feeding its own updates back."""
    ours = tuple(p.clone() for p in initial)
    theirs = tuple(p.clone() for p in initial)
    losses, worst, failures = [], {"loss": 0.0, "gradients": 0.0, "updates": 0.0}, []
    for i in range(steps):
        x, target = batches[i % len(batches)]
        expected = eager_step(theirs, x, target)
        actual = method(ours, x, target)
        try:
            errors = check_step(actual, expected)
            for kind, value in errors.items():
                worst[kind] = max(worst[kind], value)
        except AssertionError as exc:
            failures.append({"step": i, "error": str(exc).splitlines()[0]})
        losses.append(float(actual[0]))
        theirs = tuple(t.clone() for t in expected[2])
        feed_back(ours, actual[2])
    window = max(1, min(len(losses) // 5, len(batches)))
    first, last = statistics.mean(losses[:window]), statistics.mean(losses[-window:])
    return {"passed": not failures, "failure_count": len(failures), "failures": failures[:5],
            "max_absolute_error_by_kind": worst, "losses": losses, "initial_cycle_loss": first,
            "final_cycle_loss": last, "loss_decreased": last < first}, ours


def capture_loop(method: Callable, state, batches, steps: int) -> torch.cuda.CUDAGraph:
    """`steps` calls with state feedback in one CUDA graph; updates already written in place need no copy."""
    for i in range(3):
        x, target = batches[i % len(batches)]
        feed_back(state, method(state, x, target)[2])
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(steps):
            x, target = batches[i % len(batches)]
            feed_back(state, method(state, x, target)[2])
    return graph


def paired_time(graphs: dict, initial, steps: int, samples: int, warmup: int) -> dict:
    """Interleaved timing: every sample visits every method, alternating the order, resetting state outside the clock."""
    names = list(graphs)

    def reset(state):
        for dst, src in zip(state, initial):
            dst.copy_(src)

    for _ in range(warmup):
        for name in names:
            graph, state = graphs[name]
            reset(state)
            graph.replay()
    torch.cuda.synchronize()
    raw = {name: [] for name in names}
    for sample in range(samples):
        for name in (names if sample % 2 == 0 else names[::-1]):
            graph, state = graphs[name]
            reset(state)
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            end.synchronize()
            raw[name].append(start.elapsed_time(end) / steps)
    out = {}
    for name, values in raw.items():
        ordered = sorted(values)
        pick = lambda q: ordered[int(q * (len(ordered) - 1))]
        out[name] = {"median_ms": statistics.median(ordered), "p10_ms": pick(0.1), "p90_ms": pick(0.9),
                     "steps_per_second": 1e3 / statistics.median(ordered), "samples": samples,
                     "steps_per_replay": steps, "raw_ms": values}
    return out


def bootstrap_ratio(numerator: list[float], denominator: list[float], draws: int = 2000, seed: int = 0) -> dict:
    """Median-of-resample ratio of paired samples with a 95 % interval."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    a, b = torch.tensor(numerator, dtype=torch.float64), torch.tensor(denominator, dtype=torch.float64)
    picks = torch.randint(len(a), (draws, len(a)), generator=gen)
    ratios = (a[picks].median(dim=1).values / b[picks].median(dim=1).values).sort().values
    return {"median_ratio": float(ratios.median()), "ci95_ratio": [float(ratios[int(0.025 * (draws - 1))]), float(ratios[int(0.975 * (draws - 1))])],
            "draws": draws, "seed": seed}


def amortization(name: str, baseline: str, timings: dict, compile_s: dict, capture_s: dict) -> dict:
    extra = (compile_s[name] + capture_s[name]) - (compile_s[baseline] + capture_s[baseline])
    saved = timings[baseline]["median_ms"] - timings[name]["median_ms"]
    return {"baseline": baseline, "incremental_setup_seconds": extra, "steady_state_savings_ms_per_step": saved,
            "break_even_steps": max(0.0, extra * 1e3 / saved) if saved > 0 else None}


def run(args) -> dict:
    config = {k: (str(v) if isinstance(v, Path) else v) for k, v in vars(args).items()}
    result = {"status": "pending", "config": config, "optimizer": "sgd", "task": args.task,
              "numerical_policy": "FP32 master weights; BF16 compute casts; every loss, gradient and update checked against eager PyTorch",
              "numerical_tolerances": {k: {"rtol": r, "atol": a} for k, (r, a) in TOLERANCES.items()}}
    if not torch.cuda.is_available():
        result.update(status="skipped", reason="CUDA unavailable")
        return result
    device = torch.device("cuda", torch.cuda.current_device())
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    params, batches = make_problem(args.batch, args.input, args.hidden, args.output, device, args.batches, args.seed, args.task)
    example = (params, *batches[0])
    options = {} if args.max_blocks is None else {"max_blocks": args.max_blocks}

    compile_s, warm_s = {"eager_graph": 0.0}, {"eager_graph": 0.0}
    builders = {"megakernel": lambda: tk_compile(eager_step, example, **options),
                "mega_inplace": lambda: compile_training(eager_step, example, **options)}
    methods: dict[str, Callable] = {}
    for name, build in builders.items():
        start = time.perf_counter()
        methods[name] = build()
        compile_s[name] = time.perf_counter() - start                      # cold unless the cubin cache already holds this kernel
        start = time.perf_counter()
        build()
        warm_s[name] = time.perf_counter() - start                         # cubin cache hit: trace, plan, emit, load
    methods["eager_graph"] = eager_step
    result["device"] = torch.cuda.get_device_name(device)
    result["software"] = {"torch": torch.__version__, "cuda": torch.version.cuda}
    result["compilation_seconds"] = compile_s
    result["warm_compilation_seconds"] = warm_s
    kernel_keys = ("materialized_operations", "inlined_operations", "grid_barriers", "max_work_blocks", "workspace_elements",
                   "tensor_core_operations", "direct_state_commits")
    result["kernel"] = {n: {k: getattr(methods[n].runner.generated, k) for k in kernel_keys} for n in builders}
    result["resource_usage"] = {n: methods[n].runner.resource_usage() for n in builders}

    result["trajectory"], result["capture_seconds"], result["replay_correctness"] = {}, {}, {}
    graphs = {}
    for name, method in methods.items():
        report, _ = trajectory(method, params, batches, args.trajectory_steps)
        result["trajectory"][name] = report
        state = tuple(p.clone() for p in params)
        torch.cuda.synchronize()
        start = time.perf_counter()
        graph = capture_loop(method, state, batches, args.steps)
        torch.cuda.synchronize()
        result["capture_seconds"][name] = time.perf_counter() - start
        graphs[name] = (graph, state)
    # the captured state-feedback path, checked on its own against an eager loop of the same length
    expected = tuple(p.clone() for p in params)
    for i in range(args.steps):
        expected = eager_step(expected, *batches[i % len(batches)])[2]
    for name, (graph, state) in graphs.items():
        for dst, src in zip(state, params):
            dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        try:
            for a, b in zip(state, expected):
                torch.testing.assert_close(a, b, rtol=TOLERANCES["updates"][0], atol=TOLERANCES["updates"][1])
            result["replay_correctness"][name] = {"passed": True}
        except AssertionError as exc:
            result["replay_correctness"][name] = {"passed": False, "error": str(exc).splitlines()[0]}

    timings = paired_time(graphs, tuple(p.clone() for p in params), args.steps, args.samples, args.warmup)
    result["timings"] = timings
    result["speed_ratio_vs_eager_graph"] = {n: t["median_ms"] / timings["eager_graph"]["median_ms"] for n, t in timings.items()}
    result["bootstrap_vs_eager_graph"] = {n: bootstrap_ratio(timings[n]["raw_ms"], timings["eager_graph"]["raw_ms"]) for n in builders}
    result["amortization"] = {n: amortization(n, "eager_graph", timings, compile_s, result["capture_seconds"]) for n in builders}
    passed = all(result["trajectory"][n]["passed"] and result["replay_correctness"][n]["passed"] for n in builders)
    result["status"] = "ok" if passed else "error"
    return result


HELDOUT_SEEDS = (101, 211, 307)
HELDOUT_SHAPES = {"tiny-online": (4, 32, 64, 16), "online": (1, 128, 128, 16), "small": (32, 128, 256, 64), "medium": (128, 512, 1024, 256)}


def heldout_suite(args) -> dict:
    """The reference's held-out protocol (reference: docs/a100-methodology.md:34-42,
    scripts/run_train_loop_suite.sh:7-28): the four harness shapes, each on three seeds that took no part in
    choosing any option, `--samples` paired samples per run; per shape and method the figure reported is the
    MEDIAN OF THE THREE SEED MEDIANS (microseconds per step), with every seed's median and the pass/fail of its
    trajectory and replay checks beside it."""
    summary: dict = {"status": "ok", "seeds": list(HELDOUT_SEEDS), "samples": args.samples, "shapes": {}}
    for shape, (batch, input_size, hidden, output) in HELDOUT_SHAPES.items():
        per_seed = {}
        for seed in HELDOUT_SEEDS:
            one = argparse.Namespace(**{**vars(args), "batch": batch, "input": input_size, "hidden": hidden, "output": output,
                                        "seed": seed, "json": None})
            result = run(one)
            if result["status"] != "ok":
                summary["status"] = "error"
            per_seed[seed] = {"status": result["status"],
                              "median_us_per_step": {n: t["median_ms"] * 1e3 for n, t in result.get("timings", {}).items()}}
        methods = sorted({n for r in per_seed.values() for n in r["median_us_per_step"]})
        summary["shapes"][shape] = {
            "batch_input_hidden_output": [batch, input_size, hidden, output],
            "median_of_seed_medians_us": {n: sorted(r["median_us_per_step"].get(n, float("nan")) for r in per_seed.values())[len(per_seed) // 2]
                                          for n in methods},
            "per_seed": per_seed}
    return summary


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--batch", type=int, default=128)
    parser.add_argument("--input", type=int, default=512)
    parser.add_argument("--hidden", type=int, default=1024)
    parser.add_argument("--output", type=int, default=256)
    parser.add_argument("--batches", type=int, default=4)
    parser.add_argument("--steps", type=int, default=20, help="steps per captured graph")
    parser.add_argument("--trajectory-steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--samples", type=int, default=30)
    parser.add_argument("--seed", type=int, default=20261025)
    parser.add_argument("--task", choices=("regression", "classification-head"), default="regression")
    parser.add_argument("--max-blocks", type=int, default=None)
    parser.add_argument("--json", type=Path)
    parser.add_argument("--heldout", action="store_true",
                        help="run the four harness shapes on the three held-out seeds and report the median of the seed medians")
    args = parser.parse_args(argv)
    counts = (args.batch, args.input, args.hidden, args.output, args.batches, args.steps, args.trajectory_steps, args.warmup, args.samples)
    if any(value < 1 for value in counts):
        parser.error("all sizes and iteration counts must be positive")
    try:
        result = heldout_suite(args) if args.heldout else run(args)
    except Exception as exc:  # the JSON records the failure, as the harness is run unattended
        import traceback
        result = {"status": "error", "error": f"{type(exc).__name__}: {exc}", "traceback": traceback.format_exc()}
    text = json.dumps(result, indent=2, sort_keys=True)
    print(text)
    if args.json:
        args.json.parent.mkdir(parents=True, exist_ok=True)
        args.json.write_text(text + "\n")
    return int(result["status"] == "error")


if __name__ == "__main__":
    raise SystemExit(main())
