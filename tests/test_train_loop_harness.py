"""The training-loop comparison harness (reference: benchmarks/train_loop.py)."""
import json

import pytest
import torch

from trainkernel_b200.benchmarks import train_loop


def test_problem_is_seeded_and_bf16_representable():
    a, batches_a = train_loop.make_problem(4, 8, 16, 4, "cpu", 2, 7, "regression")
    b, batches_b = train_loop.make_problem(4, 8, 16, 4, "cpu", 2, 7, "regression")
    assert all(torch.equal(p, q) for p, q in zip(a, b))
    assert all(torch.equal(x, y) and torch.equal(s, t) for (x, s), (y, t) in zip(batches_a, batches_b))
    assert all(p.dtype == torch.float32 and torch.equal(p, p.to(torch.bfloat16).float()) for p in a)
    assert [tuple(p.shape) for p in a] == [(8, 16), (16,), (16, 4), (4,)]
    _, heads = train_loop.make_problem(4, 8, 16, 4, "cpu", 1, 7, "classification-head")
    onehot = heads[0][1].float()
    assert torch.equal(onehot.sum(dim=1), torch.ones(4)) and set(onehot.unique().tolist()) <= {0.0, 1.0}


def test_step_gate_accepts_itself_and_rejects_a_wrong_update():
    params, batches = train_loop.make_problem(4, 8, 16, 4, "cpu", 1, 3, "regression")
    expected = train_loop.eager_step(params, *batches[0])
    assert train_loop.check_step(expected, expected) == {"loss": 0.0, "gradients": 0.0, "updates": 0.0}
    wrong = (expected[0], expected[1], tuple(p + 1e-2 for p in expected[2]))
    with pytest.raises(AssertionError, match="updates"):
        train_loop.check_step(wrong, expected)


def test_bootstrap_and_amortization_arithmetic():
    ratio = train_loop.bootstrap_ratio([1.0, 1.1, 0.9, 1.0], [2.0, 2.2, 1.8, 2.0], draws=200)
    assert 0.4 <= ratio["ci95_ratio"][0] <= ratio["median_ratio"] <= ratio["ci95_ratio"][1] <= 0.62
    timings = {"fast": {"median_ms": 1.0}, "slow": {"median_ms": 3.0}}
    paid = train_loop.amortization("fast", "slow", timings, {"fast": 4.0, "slow": 0.0}, {"fast": 0.5, "slow": 0.5})
    assert paid["break_even_steps"] == pytest.approx(2000.0)
    never = train_loop.amortization("slow", "fast", timings, {"fast": 0.0, "slow": 1.0}, {"fast": 0.0, "slow": 0.0})
    assert never["break_even_steps"] is None


def test_without_a_gpu_the_harness_reports_skipped(capsys, tmp_path):
    if torch.cuda.is_available():
        pytest.skip("CPU-only behaviour")
    code = train_loop.main(["--batch", "4", "--input", "8", "--hidden", "16", "--output", "4", "--json", str(tmp_path / "r.json")])
    assert code == 0
    assert json.loads((tmp_path / "r.json").read_text())["status"] == "skipped"
    with pytest.raises(SystemExit):
        train_loop.main(["--batch", "0"])


@pytest.mark.gpu
@pytest.mark.parametrize("task", ["regression", "classification-head"])
def test_harness_end_to_end_on_the_gpu(task, tmp_path):
    code = train_loop.main(["--batch", "32", "--input", "128", "--hidden", "256", "--output", "64", "--task", task,
                            "--samples", "5", "--warmup", "2", "--trajectory-steps", "20", "--json", str(tmp_path / "r.json")])
    report = json.loads((tmp_path / "r.json").read_text())
    assert code == 0 and report["status"] == "ok", report.get("error")
    for name in ("megakernel", "mega_inplace"):
        assert report["trajectory"][name]["passed"] and report["replay_correctness"][name]["passed"]
        assert report["timings"][name]["median_ms"] > 0
    assert report["kernel"]["mega_inplace"]["direct_state_commits"] == 4
