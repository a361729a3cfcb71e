"""Address arithmetic of the in-kernel gradient exchange, restated on the host.

The device code (`tk::st_row_scatter`, `tk::exchange_mean_item`, `tk::exchange_mean_mc_item`) and the
planner must agree on where a contribution is staged and who reduces it.  These tests walk the same
formulas in Python for world sizes 2, 4 and 8 and ragged value sizes, and check the planner's region
sizes against them: every element of every source rank lands in exactly one staging slot of exactly
one owner, inside the region the planner reserved, and the owners' items cover every chunk once.
"""
import pytest

from trainkernel_b200.plan import THREADS

CHUNK_BYTES = THREADS * 16
CHUNKS_PER_ITEM = 8


def owned_bytes(numel: int, element: int, world: int) -> int:
    chunks = -(-max(1, numel) * element // CHUNK_BYTES)
    return -(-chunks // world) * CHUNK_BYTES


def staged_address(e: int, element: int, world: int, source: int, numel: int) -> tuple[int, int]:
    """(owner rank, byte offset inside the owner's staging region) of element e contributed by `source`."""
    per_chunk = CHUNK_BYTES // element
    chunk = e // per_chunk
    return chunk % world, source * owned_bytes(numel, element, world) + ((chunk // world) * per_chunk + e % per_chunk) * element


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("numel,element", [(1, 4), (7, 2), (1536, 2), (1537, 2), (8192, 2), (8 * 1536 * 8 + 5, 2), (100_003, 4)])
def test_scatter_staging_is_a_bijection_inside_the_reserved_region(world, numel, element):
    region = world * owned_bytes(numel, element, world)
    seen: dict[tuple[int, int], tuple[int, int]] = {}
    step = max(1, numel // 4000)                       # every element for small values, a dense sample otherwise
    for e in list(range(0, numel, step)) + [numel - 1]:
        for source in range(world):
            owner, offset = staged_address(e, element, world, source, numel)
            assert 0 <= offset and offset + element <= region
            assert seen.setdefault((owner, offset), (e, source)) == (e, source)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("numel,element", [(1, 4), (1536, 2), (1537, 2), (8192 * 8192, 2), (4096 * 8192, 2), (8192, 2), (100_003, 4)])
def test_owner_items_cover_every_chunk_exactly_once(world, numel, element):
    per_chunk = CHUNK_BYTES // element
    chunks = -(-numel // per_chunk)
    items = max(1, -(-(-(-chunks // world)) // CHUNKS_PER_ITEM))         # the planner's item count of an exchange unit
    covered = []
    for rank in range(world):
        for item in range(items):
            for slot in range(item * CHUNKS_PER_ITEM, (item + 1) * CHUNKS_PER_ITEM):
                owned = slot * world + rank                               # the chunk a rank's slot-th owned chunk is
                if owned < chunks:
                    covered.append(owned)
                    # the owner reads slot `slot` of every source's staging stripe: inside the stripe
                    assert (slot + 1) * CHUNK_BYTES <= owned_bytes(numel, element, world)
    assert sorted(covered) == list(range(chunks))


def test_planner_reserves_what_the_device_formulas_need():
    import torch
    import trainkernel_b200 as tk
    from trainkernel_b200 import workloads
    from trainkernel_b200.codegen import plan_program
    from trainkernel_b200.passes import insert_gradient_exchange
    from trainkernel_b200.plan import ELEMENT_BYTES
    work = workloads.mlp_workload("w", (96, 200, 72), 32, seed=0, resident=1)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    for world in (2, 4, 8):
        plan = plan_program(insert_gradient_exchange(program, 4), inplace_outputs={5 + i: i for i in range(4)}, world=world)
        regions = []
        for unit in plan.units:
            if unit.kind != "exchange":
                continue
            source, result = unit.root.inputs[0].buffer, unit.root.output.buffer
            numel = 1
            for extent in plan.shapes[source]:
                numel *= extent
            element = ELEMENT_BYTES[plan.dtypes[source]]
            kind, offset, stripe = plan.storage[source]
            assert kind == "scatter" and stripe == owned_bytes(numel, element, world)
            regions.append((offset, offset + world * stripe))
            regions.append((plan.storage[result][1], plan.storage[result][1] + numel * element))
            chunks = -(-numel * element // CHUNK_BYTES)
            assert unit.items == max(1, -(-(-(-chunks // world)) // CHUNKS_PER_ITEM))
        regions.sort()
        assert regions[0][0] >= 4096 and regions[-1][1] <= plan.symmetric_bytes
        assert all(a[1] <= b[0] for a, b in zip(regions, regions[1:]))        # no two regions overlap
