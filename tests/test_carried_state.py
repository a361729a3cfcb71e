"""Host-side bookkeeping for values a kernel carries between launches (`runtime.CarriedState`), on CPU tensors.

The kernel may skip re-casting its FP32 masters only when NOTHING touched them since its own previous launch;
the decision is made here from tensor addresses, PyTorch version counters and the module's launch count."""
import torch

from trainkernel_b200.runtime import TRUST_CARRIED, CarriedState


class _Module:
    def __init__(self):
        self.count = 0

    def launches(self):
        return self.count


def _launch(carried, module, targets):
    """What CompiledProgram._launch does around the kernel launch."""
    flags = carried.flags(targets)
    module.count += 1
    torch.autograd.graph.increment_version(targets)
    carried.launched(targets)
    return flags


def test_trust_requires_untouched_state_same_tensors_and_no_foreign_launch():
    module = _Module()
    carried = CarriedState(64, torch.device("cpu"), module)
    a, b = torch.zeros(8), torch.zeros(8)
    assert _launch(carried, module, [a, b]) == 0                    # first launch: nothing to trust
    assert _launch(carried, module, [a, b]) == TRUST_CARRIED        # untouched since
    a.add_(1.0)                                                     # an in-place edit PyTorch counts
    assert _launch(carried, module, [a, b]) == 0
    assert _launch(carried, module, [a, b]) == TRUST_CARRIED
    c = a.clone()                                                   # another tensor in the same role
    assert _launch(carried, module, [c, b]) == 0
    assert _launch(carried, module, [c, b]) == TRUST_CARRIED
    module.count += 1                                               # somebody else launched this module (C ABI, another wrapper)
    assert _launch(carried, module, [c, b]) == 0
    assert _launch(carried, module, [c, b]) == TRUST_CARRIED
    carried.invalidate()                                            # a write the counters cannot see, declared by the caller
    assert _launch(carried, module, [c, b]) == 0
    b.data.mul_(2.0)                                                # `.data` edits are exactly such a write: still trusted
    assert _launch(carried, module, [c, b]) == TRUST_CARRIED        # ... which is why invalidate() exists
