"""Batch-sharded data parallelism for a compiled training step (one process per GPU).

The reference has no distributed code (reference: README.md:128).  This module
adds the one exchange a batch-sharded step needs: every rank runs the
*gradient half* of the program on its rows of the batch, the gradients (and
the loss) are averaged across ranks, and every rank runs the identical
*update half* on identical inputs, so replicas stay bit-identical.  Because
each rank's loss is a mean over its own rows and shards are equal-sized, the
average of the local gradients is the full-batch gradient.

`reduce="nccl"` launches the two halves as separate kernels with one
`torch.distributed.all_reduce(AVG)` over a flat gradient buffer (plus one over
the scalar loss) between them — a CUDA-graph-capturable sequence on one stream.
When the FP32 gradients are widenings of BF16 values, which is what a
BF16-compute step produces, the BF16 values are what is exchanged
(`exchange="narrow"`): half the bytes, and the averaged gradient is rounded to
BF16 once more, as the full-batch step rounds its own gradient.
"""
from __future__ import annotations

from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist
from torch.utils._pytree import tree_flatten, tree_unflatten

from . import runtime
from .frontend import capture
from .passes import split_at_gradients


class PeerFailure(RuntimeError):
    """A peer rank reported a failure, or gave no sign of life within the limit."""

    def __init__(self, rank: int, reason: str) -> None:
        super().__init__(f"trainkernel: rank {rank} failed: {reason}")
        self.rank = rank
        self.reason = reason


class PeerHealth:
    """Host-side liveness of the ranks of a sharded step, kept in a `torch.distributed` key-value store.

    The step kernels of all ranks wait for each other's flags on the device (bounded, two seconds by
    default, after which the launch is lost and every rank has to reset).  It is cheaper to learn on the
    HOST that a peer is gone and not launch at all: every rank calls `arrive(step)` when it is about to
    launch step `step`, and `wait_for_peers(step)` returns once every rank has arrived at that step, or
    raises `PeerFailure` naming the rank that reported a failure (`report_failure`, typically from an
    `except` block) or that stayed silent for `timeout_s`.  Nothing here touches a GPU.
    """

    def __init__(self, store, rank: int, world: int, *, timeout_s: float = 5.0, prefix: str = "trainkernel/health") -> None:
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix = timeout_s, prefix

    def arrive(self, step: int) -> None:
        self.store.set(f"{self.prefix}/step/{self.rank}", str(int(step)))

    def report_failure(self, reason: str) -> None:
        self.store.set(f"{self.prefix}/failed/{self.rank}", str(reason) or "unspecified")

    def failed_peer(self) -> tuple[int, str] | None:
        for peer in range(self.world):
            key = f"{self.prefix}/failed/{peer}"
            if peer != self.rank and self.store.check([key]):
                return peer, self.store.get(key).decode()
        return None

    def wait_for_peers(self, step: int) -> None:
        import time
        deadline = time.monotonic() + self.timeout_s
        waiting = [peer for peer in range(self.world) if peer != self.rank]
        while True:
            failed = self.failed_peer()
            if failed is not None:
                raise PeerFailure(*failed)
            still = []
            for peer in waiting:
                key = f"{self.prefix}/step/{peer}"
                if not self.store.check([key]) or int(self.store.get(key).decode()) < step:
                    still.append(peer)
            waiting = still
            if not waiting:
                return
            if time.monotonic() > deadline:
                raise PeerFailure(waiting[0], f"no sign of life for {self.timeout_s:g} s while waiting for step {step}")
            time.sleep(0.002)


def shard_rows(batch: int, rank: int, world: int) -> slice:
    """Rows of the global batch owned by `rank`; the batch must divide evenly."""
    if batch % world:
        raise ValueError("trainkernel: global batch must divide evenly across ranks")
    per = batch // world
    return slice(rank * per, (rank + 1) * per)


class ShardedTrainingStep:
    """`(state, *data) -> (loss, grads, state)` with gradients averaged over a process group.

    `example_inputs` hold this rank's shard.  State tensors are updated in
    place, as with `compile_training`.  The returned loss and gradients are the
    cross-rank averages and live in buffers owned by this object (reused by the
    next call).
    """

    def __init__(self, fn: Callable[..., Any], example_inputs: Sequence[Any], *, group: Any = None,
                 reduce: str = "nccl", exchange: str = "auto", **options: Any) -> None:
        if reduce != "nccl":
            raise ValueError("trainkernel: reduce must be 'nccl'")
        if exchange not in ("auto", "float32", "narrow"):
            raise ValueError("trainkernel: exchange must be 'auto', 'float32' or 'narrow'")
        if "inplace_outputs" in options:
            raise ValueError("trainkernel: the sharded step derives its own state mapping")
        self.group = group
        program, output_tree = capture(fn, example_inputs)
        flat, self.input_tree = tree_flatten(tuple(example_inputs))
        state_leaves, _ = tree_flatten(example_inputs[0])
        n = self.count = len(state_leaves)
        self.output_tree = output_tree
        self.program = program
        # "narrow": exchange the 16-bit values the FP32 gradients are widened from (half the bytes).
        self.narrow = False
        if exchange in ("auto", "narrow"):
            try:
                gradient_half, update_half = split_at_gradients(program, n, narrow_exchange=True)
                self.narrow = True
            except ValueError:
                if exchange == "narrow":
                    raise
        if not self.narrow:
            gradient_half, update_half = split_at_gradients(program, n)
        self.gradient = runtime.compile_program(gradient_half, flat, **options)
        device = self.device = self.gradient.device
        # The loss is one FP32 word; every exchanged gradient lives back to back in one flat buffer
        # of the exchange dtype, so one collective covers them all.
        exchanged = gradient_half.outputs[1:]
        dtypes = {spec.dtype for spec in exchanged}
        if len(dtypes) != 1 or gradient_half.outputs[0].dtype != "float32":
            raise ValueError("trainkernel: the sharded step needs an FP32 loss and gradients of one dtype")
        dtype = getattr(torch, dtypes.pop())
        sizes = [spec_numel(spec.shape) for spec in exchanged]
        padded = [-(-size // 128) * 128 for size in sizes]          # keep every slice 256-byte aligned
        self.loss = torch.zeros((), dtype=torch.float32, device=device)
        self.flat = torch.zeros(sum(padded), dtype=dtype, device=device)
        self.views = []
        cursor = 0
        for spec, size, pad in zip(exchanged, sizes, padded):
            self.views.append(self.flat[cursor:cursor + size].view(spec.shape))
            cursor += pad
        update_inputs = tuple(state_leaves) + tuple(self.views)
        offset = n if self.narrow else 0                              # narrow: outputs are (grads..., updated...)
        self.update = runtime.compile_program(update_half, update_inputs,
                                              inplace_outputs={offset + i: i for i in range(n)}, **options)
        self.gradients = None
        if self.narrow:
            self.gradients = tuple(torch.empty(spec.shape, dtype=getattr(torch, spec.dtype), device=device)
                                   for spec in update_half.outputs[:n])
        self.gradient_workspace = torch.empty(self.gradient.generated.workspace_elements, dtype=torch.float32, device=device)
        self.update_workspace = torch.empty(self.update.generated.workspace_elements, dtype=torch.float32, device=device)

    @property
    def kernels_per_step(self) -> int:
        return 2

    def __call__(self, *args: Any):
        flat, tree = tree_flatten(args)
        if tree != self.input_tree:
            raise ValueError("trainkernel: runtime input pytree differs from the compiled signature")
        flat = tuple(flat)
        self.gradient._validate_inputs(flat)
        state = flat[:self.count]
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self.gradient.module.launch(self.gradient.launch_inputs(flat), (self.loss, *self.views), self.gradient_workspace, stream)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.AVG, group=self.group)
            dist.all_reduce(self.loss, op=dist.ReduceOp.AVG, group=self.group)
        if self.narrow:
            outputs = (*self.gradients, *state)
            grads = self.gradients
        else:
            outputs = state
            grads = tuple(self.views)
        self.update.module.launch(self.update.launch_inputs(state + tuple(self.views)), outputs, self.update_workspace, stream)
        torch.autograd.graph.increment_version(list(state))
        return tree_unflatten([self.loss, *grads, *state], self.output_tree)

    def status(self) -> None:
        self.gradient.status()
        self.update.status()

    def close(self) -> None:
        """Wait for this rank's work and drop the kernels and buffers (call before the process group goes away)."""
        torch.cuda.synchronize(self.device)
        self.gradient = self.update = None
        self.flat = self.views = self.gradients = None


def spec_numel(shape: tuple[int, ...]) -> int:
    total = 1
    for extent in shape:
        total *= extent
    return total


class _Pointer:
    """Raw device address with the one method the launcher needs."""

    def __init__(self, address: int) -> None:
        self.address = int(address)

    def data_ptr(self) -> int:
        return self.address


class FusedShardedTrainingStep:
    """Batch-sharded training step as ONE kernel per rank with the gradient exchange inside it.

    `passes.insert_gradient_exchange` puts an `allreduce` (mean over ranks) behind the loss and
    behind every gradient; the planner turns each into an exchange unit that shares a stage with
    the next backward GEMMs.  The exchanged values live in a peer-mapped buffer allocated through
    `torch.distributed._symmetric_memory`; chunk c of a value is owned by rank c % world: every
    rank's producer (the dW GEMM epilogue, a reduction finish) writes its contribution to that chunk
    straight into the owner's staging area over NVLink, the owner sums the staged contributions from
    its own memory and pushes the mean into every rank's buffer.  Remote memory is only written.
    When the buffer also has an NVSwitch multicast mapping (`multicast=None`: use it from four ranks up if every rank has
    one; `False`: never; `True`: require it) contributions stay in their rank's own buffer instead:
    the owner of a chunk reads the in-switch sum with `multimem.ld_reduce` and delivers the mean to all
    ranks with one `multimem.st`, which halves the bytes each rank's links carry.
    Ranks order themselves with epoch flags stored into each other's buffer after grid barriers.
    All ranks must launch the step the same number of times; state is updated in place and the
    returned loss and gradients are the cross-rank means (buffers owned by this object).
    """

    # Smallest world size at which the multicast form is preferred when available.  With two ranks it
    # moves more bytes per link than scattering does (every multimem access also loops through the
    # switch for the issuing rank's own copy), but with stream warps issuing its loads beside the GEMM
    # tiles it is the faster form there too: measured on two B200s, one call, ms per step: multicast with
    # stream warps 4.30, peer stores without 4.43, peer stores with 4.50, multicast without 4.81.
    MULTICAST_FROM = 2
    # Smallest world size at which every block of the PEER-STORE form gets stream warps (four more warps that run
    # the exchange and the FP32 updates of a stage beside its GEMM tiles); the multicast form always has them.
    # Measured on B200 with the medium MLP: at four ranks the step takes 2.75 ms with them and 3.12 ms without;
    # at two ranks the peer-store form takes 4.50 ms with them and 4.43 ms without.
    STREAM_WARPS_FROM = 4

    def __init__(self, fn: Callable[..., Any], example_inputs: Sequence[Any], *, group: Any = None,
                 multicast: bool | None = None, health: PeerHealth | None = None, **options: Any) -> None:
        from .codegen import generate
        self.group = group
        self.health = health
        self.steps_launched = 0
        from .passes import insert_gradient_exchange
        if "inplace_outputs" in options or "world" in options:
            raise ValueError("trainkernel: the sharded step derives its own state mapping and world size")
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        program, self.output_tree = capture(fn, example_inputs)
        flat, self.input_tree = tree_flatten(tuple(example_inputs))
        state_leaves, _ = tree_flatten(example_inputs[0])
        n = self.count = len(state_leaves)
        if not flat or any(t.device.type != "cuda" for t in flat):
            raise RuntimeError("trainkernel: CUDA sm_100a GPU required; CPU IR inspection is available through capture()")
        device = self.device = flat[0].device
        self.program = insert_gradient_exchange(program, n)
        verbose = options.pop("verbose", False)
        # with peers, every block gets stream warps: they run the exchange and the FP32 updates of a stage while
        # the other warps run its GEMM tiles
        asked = options.pop("background", None)

        def stream_warps(through_the_switch: bool) -> bool:
            if asked is not None:
                return bool(asked)
            return self.world > 1 if through_the_switch else self.world >= self.STREAM_WARPS_FROM

        inplace = {1 + n + i: i for i in range(n)}
        # The size of the symmetric buffer depends on the exchange form, and whether the multicast form
        # is available is only known once a buffer has been mapped: plan both, allocate for the larger.
        self.generated = generate(self.program, inplace_outputs=inplace, world=self.world, background=stream_warps(False), **options)
        words = self.generated.symmetric_bytes // 4
        through_switch = None
        if multicast is None:
            multicast = None if self.world >= self.MULTICAST_FROM else False
        if self.world > 1 and multicast is not False:
            through_switch = generate(self.program, inplace_outputs=inplace, world=self.world, multicast=True,
                                      background=stream_warps(True), **options)
            words = max(words, through_switch.symmetric_bytes // 4)
        # the peer-mapped buffer: header words (epoch, rank, barrier flags) then the exchanged values
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.symmetric = symm_mem.empty(words, dtype=torch.int32, device=device)
            self.symmetric.zero_()
            self.symmetric[1] = self.rank
            torch.cuda.synchronize(device)
            handle = symm_mem.rendezvous(self.symmetric, group if group is not None else dist.group.WORLD)
            self._handle = handle
            peers = [int(p) for p in handle.buffer_ptrs]
            switch_pointer = int(getattr(handle, "multicast_ptr", 0) or 0)
            # every rank must take the same form: use the switch only if all ranks got a multicast mapping
            agreed = torch.tensor([1 if switch_pointer else 0], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            if through_switch is not None and int(agreed.item()):
                self.generated = through_switch
            elif multicast:
                raise RuntimeError("trainkernel: multicast exchange requested but the symmetric buffer has no multicast mapping")
            dist.barrier(group)
        else:
            self.symmetric = torch.zeros(words, dtype=torch.int32, device=device)
            peers = [self.symmetric.data_ptr()]
            switch_pointer = 0
        self.multicast = self.generated.multicast
        self._extra = [_Pointer(self.symmetric.data_ptr())] + [_Pointer(p) for p in peers]
        if self.multicast:
            self._extra.append(_Pointer(switch_pointer))
        cubin = runtime.build_cubin(self.generated.source, verbose=verbose)
        with torch.cuda.device(device):
            torch.cuda.current_stream(device)
            self.module = runtime._Module(self.generated, cubin, device)
        self._checker = runtime.CompiledProgram(program, self.generated, self.module, device, {1 + n + i: i for i in range(n)})
        self.carried = self._checker.carried
        self.loss = torch.zeros((), dtype=torch.float32, device=device)
        self.gradients = tuple(torch.empty(spec.shape, dtype=getattr(torch, spec.dtype), device=device)
                               for spec in program.outputs[1:1 + n])
        self.workspace = torch.empty(self.generated.workspace_elements, dtype=torch.float32, device=device)

    @property
    def kernels_per_step(self) -> int:
        return 1

    def __call__(self, *args: Any):
        flat, tree = tree_flatten(args)
        if tree != self.input_tree:
            raise ValueError("trainkernel: runtime input pytree differs from the compiled signature")
        flat = tuple(flat)
        self._checker._validate_inputs(flat)
        if self.health is not None and not torch.cuda.is_current_stream_capturing():
            # learn on the host that a peer is gone instead of launching a kernel that would wait for it
            self.health.arrive(self.steps_launched)
            self.health.wait_for_peers(self.steps_launched)
        self.steps_launched += 1
        state = flat[:self.count]
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if self.carried is not None:
            self.module.launch((*flat, *self._extra, self.carried.buffer), (self.loss, *self.gradients, *state), self.workspace, stream,
                               self.carried.flags(state))
        else:
            self.module.launch((*flat, *self._extra), (self.loss, *self.gradients, *state), self.workspace, stream)
        torch.autograd.graph.increment_version(list(state))
        if self.carried is not None:
            self.carried.launched(state)
        return tree_unflatten([self.loss, *self.gradients, *state], self.output_tree)

    def status(self) -> None:
        self._checker.status()

    def check(self) -> None:
        """Collective status check: every rank synchronises, the ranks agree on whether ANY of them saw a
        timed-out wait, and if so ALL of them reset (kernel status words, barrier words, the epoch and flag
        words of the peer-mapped header) before `RuntimeError` is raised on every rank.  A kernel that
        gave up leaves partial outputs and an epoch that differs from its peers', so one rank cannot
        recover alone.  Call it every few steps of a long loop; it costs a device synchronisation."""
        message = ""
        try:
            self._checker.status()
        except RuntimeError as error:
            message = str(error)
        failed = torch.tensor([1 if message else 0], dtype=torch.int32, device=self.device)
        if self.world > 1:
            dist.all_reduce(failed, op=dist.ReduceOp.MAX, group=self.group)
        if not int(failed.item()):
            return
        self.recover()
        raise RuntimeError(message or "trainkernel: a peer rank's step kernel reported a timed-out wait; all ranks were reset")

    def recover(self) -> None:
        """Reset this rank's kernel state and exchange header; every rank must call it at the same point."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)
        self.module.lib.tk_module_reset(self.module.handle)
        if self.carried is not None:
            self.carried.invalidate()
        header = self.symmetric[:1024]
        header.zero_()
        self.symmetric[1] = self.rank
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)

    def close(self) -> None:
        """Wait for this rank's work, then release the kernel, the rendezvous handle and the peer-mapped
        buffer, in that order.  Every rank should call it (followed by a barrier) before the process
        group is destroyed or the process exits, so that no rank's memory disappears while a peer still
        has it mapped or bound to the switch's multicast object."""
        torch.cuda.synchronize(self.device)
        self.module = None
        self._checker = None
        self.carried = None
        self._extra = []
        self._handle = None
        self.symmetric = None
