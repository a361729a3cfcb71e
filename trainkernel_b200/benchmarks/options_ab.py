"""A/B of code-generation options on one GPU, inside ONE process.

GPUs of one pool differ by several per cent under a power cap, and so do two runs on the same GPU,
so a generator option is judged only against its alternative in the same process: every variant
compiles the same training step with its own options, captures a 20-step CUDA graph with state
feedback, and the graphs are replayed in interleaved rounds under CUDA events.  Reported per
workload and variant: the median and the minimum time per step in microseconds, and whether the
variant's final state is bit-identical to the first variant's (every variant replays the same
number of steps from the same seeded state; options that only move work around must agree to the
bit, options that change a summation order need not).

    python -m trainkernel_b200.benchmarks.options_ab 'four={"wide_epilogue":false};eight=' c4,c3,c2
    python -m trainkernel_b200.benchmarks.options_ab 'deep={"simt_depth":128};auto=' mlp-32-64-16@4,gemv

A variant is `name=` followed by a JSON object of `codegen.generate` options (empty: the defaults);
a workload is one of `workloads.CONFIG_NAMES` or `mlp-<in>-<hidden>-...-<out>@<batch>`.
`--build-only` generates and compiles the kernels without a GPU (nvcc cross-compiles), so that a
later run on a GPU finds them in the cache.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from .. import capture, codegen, compile_training, runtime, workloads

GRAPH_STEPS = 20


def parse_variants(text: str) -> dict[str, dict]:
    variants: dict[str, dict] = {}
    for item in text.split(";"):
        name, _, options = item.partition("=")
        if not name:
            raise ValueError("trainkernel: a variant needs a name")
        variants[name] = json.loads(options) if options else {}
    return variants


def build_workload(name: str, device: str = "cpu") -> workloads.Workload:
    if name.startswith("mlp-"):
        sizes, _, batch = name[4:].partition("@")
        return workloads.mlp_workload(name, tuple(int(v) for v in sizes.split("-")), int(batch), seed=0, device=device)
    return workloads.build(name, device=device)


def build_only(variants: dict[str, dict], names: list[str]) -> None:
    for name in names:
        work = build_workload(name)
        program, _ = capture(work.fn(), (work.state, *work.batches[0]))
        count = len(work.state) if isinstance(work.state, tuple) else 1
        inplace = {1 + count + i: i for i in range(count)}
        for variant, options in variants.items():
            runtime.build_cubin(codegen.generate(program, inplace_outputs=inplace, **options).source)
            print(json.dumps({"workload": name, "variant": variant, "built": True}), flush=True)


def measure(variants: dict[str, dict], names: list[str], rounds: int, replays: int) -> None:
    for name in names:
        graphs = {}
        for variant, options in variants.items():
            work = build_workload(name, device="cuda")
            compiled = compile_training(work.fn(), (work.state, *work.batches[0]), **options)
            for i in range(3):
                compiled(work.state, *work.batches[i % len(work.batches)])
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(GRAPH_STEPS):
                    compiled(work.state, *work.batches[i % len(work.batches)])
            graph.replay()
            torch.cuda.synchronize()
            graphs[variant] = (graph, compiled, work)
        samples: dict[str, list[float]] = {variant: [] for variant in variants}
        for _ in range(rounds):
            for variant in variants:
                graph = graphs[variant][0]
                for _ in range(replays):
                    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    begin.record()
                    graph.replay()
                    end.record()
                    end.synchronize()
                    samples[variant].append(begin.elapsed_time(end) * 1e3 / GRAPH_STEPS)
        torch.cuda.synchronize()
        first = next(iter(variants))
        state_of = {variant: graphs[variant][2].state if isinstance(graphs[variant][2].state, tuple) else (graphs[variant][2].state,)
                    for variant in variants}
        for variant in variants:
            graphs[variant][1].runner.status()
            print(json.dumps({"workload": name, "variant": variant, "options": variants[variant],
                              "us_per_step_p50": round(statistics.median(samples[variant]), 2),
                              "us_per_step_min": round(min(samples[variant]), 2), "samples": len(samples[variant]),
                              "state_equals_first_variant": all(torch.equal(a, b) for a, b in zip(state_of[variant], state_of[first]))}),
                  flush=True)
        del graphs
        torch.cuda.empty_cache()


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("variants", help="name=JSON;name=JSON... (empty JSON: default options)")
    parser.add_argument("workloads", help="comma-separated workload names")
    parser.add_argument("--rounds", type=int, default=4, help="interleaved rounds over the variants")
    parser.add_argument("--replays", type=int, default=3, help="timed graph replays per variant and round")
    parser.add_argument("--build-only", action="store_true", help="generate and compile the kernels, run nothing")
    args = parser.parse_args(argv)
    variants, names = parse_variants(args.variants), args.workloads.split(",")
    if args.build_only:
        build_only(variants, names)
    else:
        measure(variants, names, args.rounds, args.replays)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
