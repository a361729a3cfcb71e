"""Structural checks of the stage planner and the emitter (CPU only; nvcc cross-compiles)."""
from math import prod

import pytest
import torch

import trainkernel_b200 as tk
from trainkernel_b200 import codegen, runtime, workloads
from trainkernel_b200.codegen import generate, plan_program
from trainkernel_b200.plan import ELEMENT_BYTES


def _step_program(name):
    work = workloads.build(name)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    n = len(work.state) if isinstance(work.state, tuple) else 1
    return program, {1 + n + i: i for i in range(n)}


def test_tiny_mlp_schedule_shares_stages_and_commits_directly():
    program, inplace = _step_program("c2")
    g = generate(program, inplace_outputs=inplace)
    # weight shadows | fwd 1 | fwd 2 (+loss terms, dY) | dW2, dX, db2, loss | dW1, db1
    assert g.stages == 5 and g.grid_barriers == 4
    assert g.tensor_core_operations == 5
    assert g.direct_state_commits == 4 and g.staged_state_commits == 0
    assert g.direct_outputs == 9
    by_stage = {}
    for stage, kind, name, path, items in g.units:
        by_stage.setdefault(stage, []).append(name)
    assert {"mm_2", "mm_3"} <= set(by_stage[3])          # dW and dX of a layer share a stage
    # a program this small casts its weights in every launch
    assert g.carry_bytes == 0 and "carried" not in g.source
    # when asked to, the BF16 copies of W1 and W2 are carried to the next launch in two copies each (read one, write the other)
    carrying = generate(program, inplace_outputs=inplace, carry_shadows=True)
    assert carrying.carry_bytes == 2 * 2 * (128 * 256 + 256 * 128) and carrying.input_count == len(program.inputs) + 1
    assert carrying.source.count("if (!carried") == 2 and "tk_carry_phase ?" in carrying.source and carrying.stages == 5
    # one copy, rewritten in place: dW2 (mm_2), whose epilogue rewrites W2's copy, runs one stage after dX
    # (mm_3), the copy's last reader, and shares that stage with dW1 (mm_4)
    single = generate(program, inplace_outputs=inplace, carry_shadows="reorder")
    stages = {name: stage for stage, kind, name, path, items in single.units}
    assert single.carry_bytes == 2 * (128 * 256 + 256 * 128) and "tk_carry_phase" not in single.source
    assert stages["mm_3"] == 3 and stages["mm_2"] == stages["mm_4"] == 4 and single.stages == 5
    assert "tcgen05" not in g.source and "tk::gemm_tc<" in g.source   # device library is included, not pasted


def test_unfused_schedule_is_longer_and_fp32_master_update_is_fused_when_enabled():
    program, inplace = _step_program("c2")
    fused = generate(program, inplace_outputs=inplace)
    unfused = generate(program, inplace_outputs=inplace, fuse_pointwise=False, fuse_epilogues=False)
    assert fused.grid_barriers < unfused.grid_barriers
    assert unfused.inlined_operations == 0
    assert unfused.materialized_operations == len(program.operations)
    # fused: the SGD subtraction lives in the dW epilogue functor
    functor = fused.source[fused.source.index("struct Epi_mm_4"):fused.source.index("extern \"C\"")]
    assert "P.in[0]" in functor and "P.out[5]" in functor and "P.out[1]" in functor


def test_rounding_boundaries_are_kept_in_epilogues():
    program, inplace = _step_program("c2")
    g = generate(program, inplace_outputs=inplace)
    functor = g.source[g.source.index("struct Epi_mm {"):g.source.index("struct Epi_mm_1")]
    assert functor.count("tk::BF16::rnd") >= 4            # mm, bias cast, add, relu are each rounded


def test_workspace_regions_never_overlap_while_live():
    for name in ("c2", "c4"):
        program, inplace = _step_program(name)
        plan = plan_program(program, inplace_outputs=inplace)
        writer_stage, last_read = {}, {}
        for unit in plan.units:
            for store in unit.stores:
                writer_stage[store.buffer] = unit.stage
            for buffer in unit.reads:
                last_read[buffer] = max(last_read.get(buffer, -1), unit.stage)
        regions = []
        for buffer, where in plan.storage.items():
            if where[0] != "ws":
                continue
            size = max(1, prod(plan.shapes[buffer])) * ELEMENT_BYTES[plan.dtypes[buffer]]
            regions.append((where[1], where[1] + size, writer_stage[buffer], max(last_read.get(buffer, -1), writer_stage[buffer]), buffer))
            assert where[1] % 256 == 0 and where[1] + size <= plan.workspace_bytes
        for i, a in enumerate(regions):
            for b in regions[i + 1:]:
                overlap = a[0] < b[1] and b[0] < a[1]
                live_together = a[2] <= b[3] and b[2] <= a[3]
                assert not (overlap and live_together), (a, b)


def test_direct_commit_decisions():
    x = torch.randn(8, 4)
    program, _ = tk.capture(lambda x: x + 1, (x,))
    assert generate(program, inplace_outputs={0: 0}).direct_state_commits == 1
    program, _ = tk.capture(lambda x: x.t() + 1, (torch.randn(4, 4),))
    g = generate(program, inplace_outputs={0: 0})
    assert g.direct_state_commits == 0 and g.staged_state_commits == 1
    a, b = torch.randn(8, 4), torch.randn(8, 4)
    program, _ = tk.capture(lambda a, b: (b * 2.0, a + 1.0), (a, b))
    g = generate(program, inplace_outputs={0: 0, 1: 1})
    assert g.staged_state_commits >= 1                     # a swap cannot be committed in place
    # returning the old state as well forces the staged path
    program, _ = tk.capture(lambda x: (x + 1, x), (x,))
    g = generate(program, inplace_outputs={0: 0})
    assert g.direct_state_commits == 0


def test_option_and_mapping_validation():
    program, _ = tk.capture(lambda x: x + 1, (torch.randn(8),))
    with pytest.raises(ValueError, match="max_blocks"):
        generate(program, max_blocks=0)
    with pytest.raises(ValueError, match="blocks_per_sm"):
        generate(program, blocks_per_sm=9)
    with pytest.raises(ValueError, match="hopper_wgmma"):
        generate(program, hopper_wgmma=True)
    with pytest.raises(ValueError, match="invalid inplace"):
        generate(program, inplace_outputs={3: 0})
    program2, _ = tk.capture(lambda x, y: (x + 1, y + 1), (torch.randn(8), torch.randn(8)))
    with pytest.raises(ValueError, match="distinct inputs"):
        generate(program2, inplace_outputs={0: 0, 1: 0})
    program3, _ = tk.capture(lambda x: x.t(), (torch.randn(4, 4),))
    with pytest.raises(ValueError, match="computed values"):
        generate(program3, inplace_outputs={0: 0})
    assert generate(program, gemm_k_tile=16, threads_per_block=256).grid >= 1   # reference geometry knobs are ignored


def test_path_selection():
    def paths(fn, *tensors, **options):
        program, _ = tk.capture(fn, tensors)
        return [u[3] for u in generate(program, **options).units if u[1] == "gemm"]
    bf = torch.bfloat16
    assert paths(lambda a, b: a @ b, torch.randn(128, 64).to(bf), torch.randn(64, 64).to(bf)) == ["tc"]
    assert paths(lambda a, b: a @ b, torch.randn(128, 64).to(bf), torch.randn(64, 64).to(bf), tensor_cores=False) == ["simt"]
    # a program whose largest product is below 0.6 MFLOP stays off the tensor path altogether ...
    assert paths(lambda a, b: a @ b, torch.randn(64, 64).to(bf), torch.randn(64, 64).to(bf)) == ["simt"]
    # ... but one large product keeps the small ones of the same program on it
    assert paths(lambda a, b, c: (a @ b) @ c, torch.randn(128, 64).to(bf), torch.randn(64, 64).to(bf), torch.randn(64, 16).to(bf)) == ["tc", "tc"]
    assert paths(lambda a, b: a @ b, torch.randn(64, 64), torch.randn(64, 64)) == ["simt"]
    assert paths(lambda a, b: a @ b, torch.randn(17, 33).to(bf), torch.randn(33, 65).to(bf)) == ["simt"]   # 66-byte rows
    assert paths(lambda a, b: a @ b, torch.randn(1, 128).to(bf), torch.randn(128, 64).to(bf)) == ["gemv"]
    assert paths(lambda a, b: a @ b, torch.randn(64, 8).to(bf), torch.randn(8, 64).to(bf)) == ["simt"]     # k <= 8


def test_generated_source_is_deterministic_and_compiles_for_sm_100a():
    program, inplace = _step_program("c2")
    a = generate(program, inplace_outputs=inplace)
    b = generate(program, inplace_outputs=inplace)
    assert a.source == b.source
    cubin = runtime.build_cubin(a.source)
    assert cubin[:4] == b"\x7fELF"


def test_medium_mlp_plan_fits_and_uses_wide_tiles():
    sizes, batch = (4096, 8192, 8192, 8192, 4096), 8192
    state = []
    for fan_in, fan_out in zip(sizes[:-1], sizes[1:]):
        state += [torch.empty(fan_in, fan_out, device="meta"), torch.empty(fan_out, device="meta")]
    x = torch.empty(batch, sizes[0], dtype=torch.bfloat16, device="meta")
    t = torch.empty(batch, sizes[-1], dtype=torch.bfloat16, device="meta")
    program, _ = tk.capture(lambda s, x, t: workloads.mlp_master_step(s, x, t, 1e-3), (tuple(state), x, t))
    g = generate(program, inplace_outputs={9 + i: i for i in range(8)})
    assert g.tensor_core_operations == 11 and g.direct_state_commits == 8
    assert g.grid == 148 and g.workspace_bytes < 2 * 2 ** 30
    assert g.cluster == 2 and "tk::gemm_tc2<" in g.source and "tk::gemm_tc<" not in g.source   # pair tiles everywhere
    single = generate(program, inplace_outputs={9 + i: i for i in range(8)}, two_cta=False)
    assert single.cluster == 1 and "tk::gemm_tc<256" in single.source
    # 22 operand maps, 7 of them twice (the weights' BF16 copies exist in two copies); the shim's parameter block holds 8 KiB
    assert len(g.tensor_maps) == 29 and g.param_bytes <= 8192 and g.carry_bytes == 2 * 2 * 201326592


def test_exchange_units_overlap_backward_gemms_and_precede_updates():
    from trainkernel_b200.passes import insert_gradient_exchange
    program, inplace = _step_program("c2")
    exchanged = insert_gradient_exchange(program, 4)
    assert sum(op.op == "allreduce" for op in exchanged.operations) == 5          # loss + 4 gradients
    plan = plan_program(exchanged, inplace_outputs=inplace, world=2)
    by_name = {u.name: u for u in plan.units}
    assert by_name["mm_2_avg"].kind == "exchange"
    # dW2 is averaged in the stage that computes dW1; the SGD update that consumes the mean follows
    assert by_name["mm_2_avg"].stage == by_name["mm_2"].stage + 1 == by_name["mm_4"].stage
    consumer = next(u for u in plan.units if "mm_2_avg" in u.reads)
    assert consumer.stage == by_name["mm_2_avg"].stage + 1 and consumer.wait_barrier == consumer.stage - 1
    assert by_name["mm_2_avg"].wait_barrier == by_name["mm_2_avg"].stage - 1
    assert set(plan.signal_barriers) == {u.wait_barrier for u in plan.units if u.wait_barrier is not None}
    # contributions are scattered into the owner's staging area; the mean is laid out like the value
    assert plan.storage["mm_2"][0] == "scatter" and plan.storage["mm_2_avg"][0] == "sym" and plan.symmetric_bytes > 4096
    assert len(plan.direct_commits) == 4                                           # updates still commit in place
    g = generate(exchanged, inplace_outputs=inplace, world=2)
    # program inputs, this rank's symmetric buffer, both ranks' mappings of it
    assert g.input_count == len(program.inputs) + 1 + 2 and g.world == 2 and g.carry_bytes == 0
    with_carry = generate(exchanged, inplace_outputs=inplace, world=2, carry_shadows=True)      # the carry buffer comes last
    assert with_carry.input_count == len(program.inputs) + 1 + 2 + 1 and with_carry.carry_bytes > 0
    assert "tk::exchange_mean<tk::BF16, 2>" in g.source and "tk::dp_signal" in g.source and "tk::dp_wait" in g.source
    assert "tk::st_row_scatter<W, 2, __nv_bfloat16>" in g.source          # dW epilogue pushes straight to the owner
    assert runtime.build_cubin(g.source)[:4] == b"\x7fELF"
    with pytest.raises(ValueError, match="world"):
        generate(exchanged, inplace_outputs=inplace, world=9)
    # through the NVSwitch multicast mapping: contributions stay local, one more pointer, no scatter
    switch = generate(exchanged, inplace_outputs=inplace, world=2, multicast=True)
    assert switch.multicast and switch.input_count == len(program.inputs) + 1 + 2 + 1
    assert f"tk::exchange_mean_mc<tk::BF16, 2>(c, &P.in[{len(program.inputs) + 1}], P.in[{len(program.inputs) + 3}]" in switch.source
    assert "st_row_scatter" not in switch.source and "tk::dp_wait" in switch.source
    assert switch.symmetric_bytes <= g.symmetric_bytes and switch.stages == g.stages
    assert runtime.build_cubin(switch.source)[:4] == b"\x7fELF"
    assert not generate(exchanged, inplace_outputs=inplace, world=1, multicast=True).multicast    # one rank: nothing to exchange through


def test_small_programs_run_as_one_cluster_with_the_hardware_barrier():
    program, inplace = _step_program("c2")
    g = generate(program, inplace_outputs=inplace)
    assert g.barrier == "cluster" and g.grid == g.cluster == 8
    assert "tk::cluster_barrier(c);" in g.source and "tk::grid_barrier(c);" not in g.source
    wide = generate(program, inplace_outputs=inplace, cluster_barrier=False)
    assert wide.barrier == "grid" and wide.cluster == 1 and wide.grid > 8 and "tk::grid_barrier(c);" in wide.source
    one = generate(program, inplace_outputs=inplace, max_blocks=1)
    assert one.barrier == "cluster" and one.grid == one.cluster == 1
    three = generate(program, inplace_outputs=inplace, max_blocks=3)
    assert three.grid == three.cluster == 2                                        # cluster sizes are powers of two
    # enough work to fill the GPU: barrier through global memory, all SMs
    big, big_inplace = _step_program("c4")
    g4 = generate(big, inplace_outputs=big_inplace)
    assert g4.barrier == "grid" and g4.grid == 148
    assert generate(big, inplace_outputs=big_inplace, cluster_barrier=True).grid == 8
    # a kernel that exchanges with peers keeps the grid barrier (its flags are raised after grid barriers)
    from trainkernel_b200.passes import insert_gradient_exchange
    assert generate(insert_gradient_exchange(program, 4), inplace_outputs=inplace, world=2).barrier == "grid"


def _deep_mlp_program(layers: int):
    sizes = tuple([32] * (layers + 1))
    work = workloads.mlp_workload("deep", sizes, 8, seed=0, resident=1)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    n = len(work.state)
    return program, {1 + n + i: i for i in range(n)}, n


def test_fixed_size_stage_tables_are_guarded():
    """The stamp area holds 55 stages and the symmetric header 64 barrier flags per rank: a program
    beyond either limit is rejected when the kernel is generated, not when it overruns a table."""
    from trainkernel_b200.passes import insert_gradient_exchange
    program, inplace, n = _deep_mlp_program(34)
    plain = generate(program, inplace_outputs=inplace)
    assert plain.stages > codegen.MAX_STAMPED_STAGES           # fine without stamps
    with pytest.raises(ValueError, match="stage stamps cover at most"):
        generate(program, inplace_outputs=inplace, stage_stamps=True)
    exchanged = insert_gradient_exchange(program, n)
    with pytest.raises(ValueError, match="at most 64 grid barriers"):
        generate(exchanged, inplace_outputs=inplace, world=2)
    small, small_inplace, _ = _deep_mlp_program(2)
    with pytest.raises(ValueError, match="trace_stage needs"):
        generate(small, inplace_outputs=small_inplace, trace_stage=1)
    with pytest.raises(ValueError, match="trace_stage needs"):
        generate(small, inplace_outputs=small_inplace, stage_stamps=True, trace_stage=99)
    assert generate(small, inplace_outputs=small_inplace, stage_stamps=True, trace_stage=1).stages <= codegen.MAX_STAMPED_STAGES


def _medium_program(batch=8192):
    sizes = (4096, 8192, 8192, 8192, 4096)
    state = []
    for fan_in, fan_out in zip(sizes[:-1], sizes[1:]):
        state += [torch.empty(fan_in, fan_out, device="meta"), torch.empty(fan_out, device="meta")]
    x = torch.empty(batch, sizes[0], dtype=torch.bfloat16, device="meta")
    t = torch.empty(batch, sizes[-1], dtype=torch.bfloat16, device="meta")
    program, _ = tk.capture(lambda s, xx, tt: workloads.mlp_master_step(s, xx, tt, 1e-3), (tuple(state), x, t))
    return program, {1 + 8 + i: i for i in range(8)}


def test_loss_and_bias_gradient_sums_are_formed_in_gemm_epilogues():
    """In the BF16 configurations no reduce unit reads a [batch, out] tensor back from memory: the loss terms
    and dY are summed per 32-row chunk in the epilogue of the GEMM that produces them, and the reduce units
    only finish over those partial sums (reference stage replaced: trainkernel/codegen.py:443-504)."""
    programs = {name: _step_program(name) for name in ("c2", "c3", "c4")}
    programs["c5"] = _medium_program()
    for name, (program, inplace) in programs.items():
        plan = plan_program(program, inplace_outputs=inplace)
        reduces = [u for u in plan.units if u.kind == "reduce"]
        assert reduces, name
        for unit in reduces:
            # partial sums, plus at most the bias vector its fused SGD update reads
            assert any(buffer.endswith("__partials") for buffer in unit.reads), (name, unit.name, unit.reads)
            assert all(buffer.endswith("__partials") or len(plan.shapes[buffer]) <= 1 for buffer in unit.reads), (name, unit.name, unit.reads)
            assert unit.phase in ("finish", "") and unit.phase != "partial"
        hosts = [u for u in plan.units if u.kind == "gemm" and u.fused]
        assert sum(len(u.fused) for u in hosts) == len(reduces)
        for host in hosts:
            for fused in host.fused:
                m, n = host.dims
                expected = -(-m // 32) * (1 if fused.mode == "cols" else -(-n // 32))
                assert fused.parts == expected and plan.shapes[fused.scratch][0] == expected
                assert plan.storage[fused.scratch][0] == "ws"
    # the squared residual is no longer stored at all: only its partial sums leave the forward epilogue
    program, inplace = programs["c5"]
    plan = plan_program(program, inplace_outputs=inplace)
    stored = {s.buffer for u in plan.units for s in u.stores}
    assert not any(name.startswith("pow") for name in stored)
    generated = generate(program, inplace_outputs=inplace)
    assert "__shfl_xor_sync" in generated.source and "mean__partials" in generated.source
    # without epilogue fusion the reductions read their operands from memory again
    unfused = plan_program(program, inplace_outputs=inplace, fuse_epilogues=False)
    assert any(u.kind == "reduce" and u.phase == "partial" for u in unfused.units)


def test_weight_copies_are_carried_only_in_kernels_of_large_gemms():
    program, inplace = _medium_program()
    plan = plan_program(program, inplace_outputs=inplace)
    assert plan.two_cta and plan.carry_pingpong and plan.carry_bytes == 2 * 2 * 201326592
    carried = [u for u in plan.units if u.carried]
    assert len(carried) == 4 and all(u.stage == 0 and u.kind == "point" for u in carried)
    for unit in carried:                                   # read copy and written copy swap places with the phase word
        copy = unit.members[0].output.buffer
        read, written = plan.storage[copy], plan.storage[copy + "__next"]
        assert read[0] == written[0] == "carry" and (read[1], read[2]) == (written[2], written[1]) and read[1] != read[2]
    # the schedule is the one without carrying: dW and dX of a layer still share a stage
    plain = plan_program(program, inplace_outputs=inplace, carry_shadows=False)
    assert [(u.name, u.stage) for u in plan.units if u.kind == "gemm"] == [(u.name, u.stage) for u in plain.units if u.kind == "gemm"]
    small, small_inplace = _step_program("c4")
    assert plan_program(small, inplace_outputs=small_inplace).carry_bytes == 0
    with pytest.raises(ValueError, match="carry_shadows"):
        plan_program(small, inplace_outputs=small_inplace, carry_shadows="sometimes")


def test_stream_warps_take_exchanges_and_only_the_updates_the_gemms_cover():
    import re
    from trainkernel_b200.passes import insert_gradient_exchange
    program, inplace = _medium_program(batch=1024)          # one of eight ranks
    exchanged = insert_gradient_exchange(program, 8)
    g = generate(exchanged, inplace_outputs=inplace, world=8, multicast=True, background=True)
    assert g.threads == 320 and "c.warp < tk::kWorkerWarps" in g.source and "bar.sync" not in g.source
    pieces = re.findall(r"// (\S+) \((\w+)\) of stage (\d+), one 32-thread slice", g.source)
    exchanges = {name for _, kind, name, _, _ in g.units if kind == "exchange"}
    assert {name for name, kind, _ in pieces if kind == "exchange"} == exchanges      # every exchange runs in the stream warps
    stage_of = {name: stage for stage, _, name, _, _ in g.units}
    gemm_stages = {stage for stage, kind, _, path, _ in g.units if kind == "gemm"}
    streamed_updates = [name for name, kind, _ in pieces if kind == "point"]
    assert streamed_updates and all(stage_of[name] in gemm_stages for name in streamed_updates)
    # the two large updates of the tail (8192 x 8192 masters) find no GEMM long enough: plain loops by the worker warps
    large = [name for stage, kind, name, _, items in g.units if kind == "point" and items > 7000]
    assert len(large) == 2 and not set(large) & set(streamed_updates)
    everything = generate(exchanged, inplace_outputs=inplace, world=8, multicast=True, background=True, stream_everything=True)
    assert set(large) <= {name for name, kind, _ in re.findall(r"// (\S+) \((\w+)\) of stage (\d+), one 32-thread slice", everything.source)}
    # without stream warps the kernel has 192 threads and no background pieces
    plain = generate(exchanged, inplace_outputs=inplace, world=8, multicast=True)
    assert plain.threads == 192 and "32-thread slice" not in plain.source


def test_single_cta_tensor_core_kernels_get_eight_epilogue_warps():
    program, inplace = _step_program("c4")
    g = generate(program, inplace_outputs=inplace)
    # 320 threads: warps 6..9 share the TMEM lane quarters of warps 2..5; one ring slot (32 KiB at 128-wide tiles) less
    assert g.threads == 320 and "#define TK_EPI_WARPS 8" in g.source and "#define TK_RING_BN 128" in g.source
    assert g.dynamic_smem == 5 * (128 * 64 * 2 + 128 * 64 * 2) + 1024
    assert "kPipelined = true" not in g.source and "kFetchFirst = true" in g.source     # only the first chunk is fetched early
    # everything that is not a tensor-core GEMM is cut for 192 threads and keeps the extra warps out
    assert g.source.count("the four extra epilogue warps have no part in this unit") == sum(
        1 for _, kind, _, path, _ in g.units if not (kind == "gemm" and path == "tc"))
    narrow = generate(program, inplace_outputs=inplace, wide_epilogue=False)
    assert narrow.threads == 192 and "TK_EPI_WARPS" not in narrow.source and narrow.dynamic_smem == 4 * 49152 + 1024
    assert "kPipelined = true" in narrow.source
    # pair-tile kernels keep four epilogue warps unless asked; kernels without tensor-core GEMMs have nothing to widen
    medium, medium_inplace = _medium_program()
    assert generate(medium, inplace_outputs=medium_inplace).threads == 192
    asked = generate(medium, inplace_outputs=medium_inplace, wide_epilogue=True)
    assert asked.threads == 320 and asked.dynamic_smem == 5 * 32768 + 1024
    plain, plain_inplace = _step_program("c1")
    assert generate(plain, inplace_outputs=plain_inplace).threads == 192


def test_simt_gemms_stage_no_deeper_than_their_k():
    work = workloads.mlp_workload("tiny_online", (32, 64, 16), 4)
    program, _ = tk.capture(work.fn(), (work.state, *work.batches[0]))
    g = generate(program, inplace_outputs={5 + i: i for i in range(4)})
    import re
    depths = {name: int(depth) for depth, name in re.findall(r"tk::gemm_simt<(\d+), [^>]*?Epi_(\w+)>", g.source)}
    assert depths and set(depths.values()) <= {32, 64}                 # K is 32, 64, 16, 4 and 4 in this program
    assert depths["mm"] == 32 and depths["mm_1"] == 64
    forced = generate(program, inplace_outputs={5 + i: i for i in range(4)}, simt_depth=128)
    assert set(re.findall(r"tk::gemm_simt<(\d+),", forced.source)) == {"128"}
    with pytest.raises(ValueError, match="simt_depth"):
        generate(program, simt_depth=48)


def test_aligned_row_accesses_are_emitted_only_where_the_layout_proves_them():
    work = workloads.mlp_workload("tiny", (128, 256, 128), 16)
    x, target = work.batches[0]
    inplace = {5 + i: i for i in range(4)}
    program, _ = tk.capture(work.fn(), (work.state, x, target))
    g = generate(program, inplace_outputs=inplace)
    # W1, b1, W2, b2 (read by the dW / bias epilogues and written in place) and the target lean on aligned pointers;
    # x is only ever a TMA operand, whose alignment the tensor-map encoder checks
    assert g.aligned_inputs == (0, 1, 2, 3, 5) and g.aligned_workspace and g.aligned_outputs
    assert "tk::ld_row_full<" in g.source and "tk::st_row_full<" in g.source
    # the same step on a target whose rows are 132 elements apart (264 bytes: every other row starts off a 16-byte
    # boundary): its loads keep the element-wise fallback and its pointer is not constrained; the rest is unchanged.
    # (A slice that merely STARTS at an odd offset has a provable layout and an unaligned pointer: the launch refuses it.)
    sliced = torch.empty(16, 132, dtype=target.dtype)[:, :128]
    viewed, _ = tk.capture(work.fn(), (work.state, x, sliced))
    v = generate(viewed, inplace_outputs=inplace)
    assert v.aligned_inputs == (0, 1, 2, 3) and v.aligned_outputs == g.aligned_outputs
    assert v.source.count("tk::ld_row_full<") == g.source.count("tk::ld_row_full<") - 1
    # switched off, nothing is assumed and nothing is required
    off = generate(program, inplace_outputs=inplace, assume_aligned=False)
    assert not off.aligned_inputs and not off.aligned_outputs and not off.aligned_workspace and "_full<" not in off.source
