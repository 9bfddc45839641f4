"""Host-side plumbing for the two ways this path shards across GPUs (one process per GPU).

The reference has no communication layer at all; both schemes are additions around its operators.

* Dense linears: column-parallel.  Rank r holds output columns [r N/g, (r+1) N/g) of the packed
  weight, scales and zero points, runs the GEMM on its slice, and the [M, N/g] slices are
  all-gathered (`gather_columns`).
* MoE layers: expert-parallel.  Rank r owns experts [r E/g, (r+1) E/g); tokens are data-parallel.
  After a count exchange, routed rows travel to the owner of their expert with one variable-size
  all-to-all that also carries each row's expert index and routing weight (`dispatch`),
  are processed there as a top-1 problem over the local experts, and travel back with a second
  all-to-all (`combine`); the token owner then sums its k slots.

Everything here is torch.distributed (NCCL on GPUs, gloo in the CPU tests) and index arithmetic;
the arithmetic kernels are passed in by the caller, so the same code is exercised on CPU with the
oracle standing in for the CUDA operators.
"""

from __future__ import annotations

import dataclasses
import time

import torch
import torch.distributed as dist


class CollectiveTimeout(RuntimeError):
    """A collective of the library formulation did not complete before the host deadline."""


# Seconds a collective may take before the caller gets an exception instead of a hang; None waits
# for ever (the torch.distributed default behaviour).  A rank that never joins -- crashed, or stuck
# in another step -- otherwise blocks its peers inside the collective with nothing to tell them why.
DEADLINE_S: float | None = None


def _finish(work, what: str, deadline_s: float | None) -> None:
    """Waits for an asynchronous collective without blocking in the backend: the host polls the work
    handle and gives up at the deadline.  The communicator is not usable after a timeout (the
    collective may still be pending on the other ranks); the caller is expected to tear the group down."""
    limit = DEADLINE_S if deadline_s is None else deadline_s
    if limit is None:
        work.wait()
        return
    end = time.monotonic() + limit
    while not work.is_completed():
        if time.monotonic() > end:
            raise CollectiveTimeout(f"{what}: not complete after {limit:.3g} s (a rank did not join?)")
        time.sleep(0.0005)
    work.wait()   # completed: returns at once; orders the current stream behind the collective (NCCL)


# ---- dense: column-parallel -------------------------------------------------------------------------
def column_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Output columns of `rank`; every shard must stay a multiple of 64 columns (repack tile)."""
    if n % world or (n // world) % 64:
        raise ValueError(f"N={n} cannot be split into {world} shards of a multiple of 64 columns")
    width = n // world
    return rank * width, (rank + 1) * width


def shard_columns(packed, scales, zeros_packed, n: int, rank: int, world: int, source: str):
    """Column shard of a GPTQ- ([K/8, N]) or AWQ-packed ([K, N/8]) weight with its scales [G, N] and
    packed zero points [G, N/8].  Sharding happens BEFORE the Marlin repack, which each rank then
    runs on its own slice."""
    lo, hi = column_range(n, rank, world)
    if source == "gptq":
        w = packed[:, lo:hi]
    elif source == "awq":
        w = packed[:, lo // 8:hi // 8]
    else:
        raise ValueError(source)
    z = None if zeros_packed is None else zeros_packed[:, lo // 8:hi // 8].contiguous()
    return w.contiguous(), scales[:, lo:hi].contiguous(), z


def gather_columns(out_local: torch.Tensor, gathered: torch.Tensor | None = None, group=None,
                   deadline_s: float | None = None) -> torch.Tensor:
    """All-gathers [M, N/g] slices; returns the [g, M, N/g] buffer (rank-major).  `as_matrix` turns it
    into [M, N]."""
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = out_local.new_empty((world, *out_local.shape))
    # flat [g*M, N/g] view: the form every backend accepts
    work = dist.all_gather_into_tensor(gathered.view(-1, out_local.shape[-1]), out_local.contiguous(), group=group,
                                       async_op=True)
    _finish(work, "gather_columns", deadline_s)
    return gathered


def as_matrix(gathered: torch.Tensor) -> torch.Tensor:
    g, m, width = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, g * width)


# ---- MoE: expert-parallel -----------------------------------------------------------------------
@dataclasses.dataclass
class DispatchPlan:
    """Where every routed (token, slot) pair of this rank goes and how to put the answers back."""
    order: torch.Tensor        # [T*k] routes sorted by destination rank (stable), as flat route ids
    send_counts: list[int]     # rows sent to each rank
    recv_counts: list[int]     # rows received from each rank
    local_expert: torch.Tensor | None = None   # [sum(recv)] expert index on this rank of every received row
    weights: torch.Tensor | None = None        # [sum(recv)] routing weight of every received row


def experts_per_rank(num_experts: int, world: int) -> int:
    if num_experts % world:
        raise ValueError(f"{num_experts} experts cannot be split evenly over {world} ranks")
    return num_experts // world


def plan_dispatch(topk_ids: torch.Tensor, num_experts: int, group=None, deadline_s: float | None = None) -> DispatchPlan:
    """Sorts this rank's routes by owner of their expert and exchanges the per-rank row counts (the
    one place the host has to read device data: the split sizes of the payload exchange)."""
    world = dist.get_world_size(group)
    per_rank = experts_per_rank(num_experts, world)
    dest = torch.div(topk_ids.reshape(-1).to(torch.int64), per_rank, rounding_mode="floor")
    order = torch.argsort(dest, stable=True)
    send = torch.bincount(dest, minlength=world).to(torch.int64)
    recv = torch.empty_like(send)
    _finish(dist.all_to_all_single(recv, send, group=group, async_op=True), "plan_dispatch", deadline_s)
    counts = torch.stack((send, recv)).tolist()
    return DispatchPlan(order, counts[0], counts[1])


def _meta_slots(dtype: torch.dtype) -> int:
    """Elements of `dtype` that hold one 32-bit word."""
    return 4 // torch.empty((), dtype=dtype).element_size()


def dispatch(x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, num_experts: int,
             plan: DispatchPlan, group=None, deadline_s: float | None = None) -> torch.Tensor:
    """One all-to-all carrying, per route, row `route // k` of x followed by two 32-bit words (expert
    index on the owner, routing weight) packed into spare columns.  Returns the rows this rank has to
    process, [sum(recv), H], and fills `plan.local_expert` / `plan.weights`."""
    top_k = topk_ids.shape[1]
    hidden = x.shape[1]
    slots = _meta_slots(x.dtype)
    per_rank = experts_per_rank(num_experts, dist.get_world_size(group))
    out_buf = x.new_empty((plan.order.numel(), hidden + 2 * slots))
    out_buf[:, :hidden] = x[torch.div(plan.order, top_k, rounding_mode="floor")]
    meta = torch.stack(((topk_ids.reshape(-1)[plan.order].to(torch.int32) % per_rank),
                        topk_weights.reshape(-1)[plan.order].to(torch.float32).view(torch.int32)), dim=1)
    out_buf[:, hidden:] = meta.view(x.dtype).view(-1, 2 * slots)
    in_buf = x.new_empty((sum(plan.recv_counts), hidden + 2 * slots))
    _finish(dist.all_to_all_single(in_buf, out_buf, plan.recv_counts, plan.send_counts, group=group, async_op=True),
            "dispatch", deadline_s)
    meta_in = in_buf[:, hidden:].contiguous().view(torch.int32)
    plan.local_expert = meta_in[:, 0].contiguous()
    plan.weights = meta_in[:, 1].contiguous().view(torch.float32)
    return in_buf[:, :hidden].contiguous()


def combine(y: torch.Tensor, plan: DispatchPlan, group=None, deadline_s: float | None = None) -> torch.Tensor:
    """Inverse of `dispatch`: returns [T*k, H] in flat route order (row t*k + slot)."""
    back = y.new_empty((sum(plan.send_counts), y.shape[1]))
    _finish(dist.all_to_all_single(back, y.contiguous(), plan.send_counts, plan.recv_counts, group=group, async_op=True),
            "combine", deadline_s)
    out = torch.empty_like(back)
    out[plan.order] = back
    return out


def expert_parallel_layer(x, topk_ids, topk_weights, num_experts, top_k, local_experts_forward, moe_sum, group=None):
    """One MoE layer, expert-parallel.

    `local_experts_forward(rows [R, H], local_expert [R] int32, weights [R] f32) -> [R, H]` runs this rank's
    experts on the received rows (sort, two routed GEMMs with silu_and_mul between, routing weight
    applied); `moe_sum([T, k, H]) -> [T, H]` adds a token's slots.
    """
    plan = plan_dispatch(topk_ids, num_experts, group)
    rows = dispatch(x, topk_ids, topk_weights, num_experts, plan, group)
    y = local_experts_forward(rows, plan.local_expert, plan.weights)
    routed = combine(y, plan, group)
    return moe_sum(routed.view(x.shape[0], top_k, x.shape[1]))


# ---- MoE: expert-parallel on the device (peer-mapped memory, no host read-back) ---------------------
class DeviceExpertParallel:
    """One expert-parallel MoE layer per call through `infiniops_b200_ep_moe_layer`: dispatch, the
    routed GEMM pair and combine run on the device over peer-mapped arenas, the flags between the
    ranks are exchanged by the kernels themselves, and nothing is read back by the host -- so a call
    can be recorded into a CUDA graph.  This class only sets the buffers up (`peer.PeerGroup` moves
    the memory handles between the processes) and keeps them alive.

    With a world of 1 no process group is needed (`group=None`, `world=1`): the same kernels run
    with this rank as the only owner."""

    def __init__(self, weights, top_k: int, max_tokens: int, device, block: int = 64, group=None, world=None):
        from . import capi, peer

        self.capi, self.weights, self.device = capi, weights, device
        lib = capi.lib()
        if world == 1:
            self.peers, self.world, self.rank = None, 1, 0
        else:
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        capacity = max_tokens * top_k
        arena_bytes = lib.infiniops_b200_ep_arena_bytes(self.world, capacity, weights.hidden)
        ctx = capi.EpContext()
        ctx.world, ctx.rank, ctx.top_k, ctx.hidden, ctx.inter = self.world, self.rank, top_k, weights.hidden, weights.inter
        ctx.experts_per_rank, ctx.capacity, ctx.moe_block_size = weights.num_experts, capacity, block
        ctx.a_dtype, ctx.b_type_id = capi._DTYPE[weights.s13.dtype], weights.qtype
        if self.world == 1:
            self._arena = torch.zeros(arena_bytes, dtype=torch.uint8, device=device)
            self._flags = torch.zeros(64, dtype=torch.int32, device=device)
            self._ctrl = torch.zeros(8, dtype=torch.int32, device=device)
            ctx.arena[0], ctx.flags[0], ctx.ctrl = self._arena.data_ptr(), self._flags.data_ptr(), self._ctrl.data_ptr()
        else:
            self.peers = peer.PeerGroup(arena_bytes, device, group)
            off = self.peers.carve(arena_bytes)
            for r in range(self.world):
                ctx.arena[r] = self.peers.address(r, off)
                ctx.flags[r] = self.peers.peer_base[r]
            self._ctrl = self.peers.ctrl
            ctx.ctrl = self._ctrl.data_ptr()
        self.ctx = ctx
        w = weights
        cw = capi.ExpertWeightsC()
        cw.w13, cw.s13, cw.groups13 = w.w13.data_ptr(), w.s13.data_ptr(), w.s13.shape[1]
        cw.w2, cw.s2, cw.groups2 = w.w2.data_ptr(), w.s2.data_ptr(), w.s2.shape[1]
        cw.z13 = None if w.z13 is None else w.z13.data_ptr()
        cw.z2 = None if w.z2 is None else w.z2.data_ptr()
        cw.w13_interleaved = int(w.interleaved)
        self.cw = cw
        need = lib.infiniops_b200_ep_workspace_bytes(ctx)
        if need == 0:
            raise capi.Error(lib.infiniops_b200_last_error().decode())
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=device)
        self.max_tokens = max_tokens

    def __call__(self, x, topk_ids, topk_weights, out=None, stream=None):
        capi = self.capi
        if out is None:
            out = torch.empty_like(x)
        capi._check(capi.lib().infiniops_b200_ep_moe_layer(
            self.ctx, self.cw, x.data_ptr(), topk_ids.data_ptr(), topk_weights.data_ptr(), x.shape[0], out.data_ptr(),
            self.workspace.data_ptr(), self.workspace.numel(), capi._stream(stream)))
        return out

    def status(self) -> tuple[int, int, int]:
        """(GEMM scratch status, wait status, slot): all zero unless a bounded device wait ran out."""
        s = self._ctrl[3:5].tolist()
        gemm = 0
        return gemm, int(s[0]), int(s[1])

    def close(self):
        if self.peers is not None:
            self.peers.close()
