"""Multi-GPU forms of the path, one process per GPU over ``torch.distributed``.

* Dense GEMMs shard by rows of A (B replicated).  Quantization is row-local along K, so a shard is
  quantized and multiplied exactly as the same rows would be on one GPU; the only collective is the
  optional all-gather of the output shards.
* The MoE block is expert-parallel: tokens are sharded across ranks, experts are split in
  contiguous ranges; one count exchange and one all-to-all of rows each way around the local
  grouped FFN.

The exchange logic is plain ``torch.distributed`` on whatever backend the group has (NCCL on GPUs,
gloo in the CPU tests); the compute steps are passed in as callables so that the CPU tests can
exercise the exchange with a reference computation.  Nothing here exists in the reference, which is
single-GPU (no collective call anywhere in it).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


def row_shard(m: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """[start, stop) of this rank's rows: `multiple`-row tiles dealt as evenly as possible, in
    rank order (the last ranks may get one tile less; a rank can be empty when m is small)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    tiles = (m + multiple - 1) // multiple
    base, extra = divmod(tiles, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return min(first * multiple, m), min((first + count) * multiple, m)


def all_gather_rows(local: torch.Tensor, m: int, group=None, multiple: int = 128) -> torch.Tensor:
    """Concatenate the ranks' row shards (shards as dealt by `row_shard`) into the full (m, n) matrix."""
    world = dist.get_world_size(group)
    sizes = [b - a for a, b in (row_shard(m, world, r, multiple) for r in range(world))]
    if local.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError(f"shard has {local.shape[0]} rows, expected {sizes[dist.get_rank(group)]}")
    if len(set(sizes)) == 1:
        out = local.new_empty(m, *local.shape[1:])
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    # ragged shards: collectives want equal sizes, so pad to the largest shard and cut afterwards
    biggest = max(sizes)
    padded = local.new_zeros(biggest, *local.shape[1:])
    padded[: local.shape[0]] = local
    out = local.new_empty(world * biggest, *local.shape[1:])
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * biggest: r * biggest + s] for r, s in enumerate(sizes)], dim=0)


def sharded_gemm(a_shard: torch.Tensor, b: torch.Tensor, a_fmt: str, b_fmt: str, out_dtype, m: int, rowwise: bool = False,
                 gather: bool = True, group=None, gemm: Optional[Callable] = None) -> torch.Tensor:
    """`a @ b` with a's rows sharded across the group: every rank multiplies its shard, the output
    shards are all-gathered when `gather`.  `gemm` defaults to the quantized `_gemm`."""
    if gemm is None:
        from .quant.linear import _gemm as gemm
    local = gemm(a_shard, b, a_fmt, b_fmt, out_dtype, rowwise)
    return all_gather_rows(local, m, group) if gather else local


class GatheredOutput:
    """The gathered (world * m, n) output of an M-sharded GEMM as symmetric memory: every rank owns one
    copy and has its peers' copies mapped, so that the GEMM's epilogue can store each tile straight into
    all of them over NVLink (fused GEMM + all-gather, no separate collective).

    payload "bf16": the result itself.  payload "mxfp8": E4M3 codes + swizzled E8M0 scale factors of the
    result quantized along its columns - what the next block-scaled GEMM would make of the bf16 matrix
    anyway (src/quant/linear.py:72-76) at 1.03 instead of 2 bytes per element on the link.

    Two sets of buffers alternate from call to call: a rank that runs ahead into its next call stores into
    the set its peers are not reading (their reads of the previous result are ordered before their own next
    GEMM on the stream, and a rank cannot get two calls ahead of a peer past the per-call rendezvous)."""

    def __init__(self, m: int, n: int, group=None, payload: str = "bf16"):
        import torch.distributed._symmetric_memory as symm
        from . import ops
        if payload not in ("bf16", "mxfp8"):
            raise ValueError(f"unknown payload {payload!r}")
        if payload == "mxfp8" and (m % 128 or n % 128):
            raise ValueError("the MXFP8 payload needs m % 128 == 0 and n % 128 == 0")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.m, self.n, self.payload = m, n, payload
        dev = torch.device("cuda", torch.cuda.current_device())
        rows = self.world * m
        self.bufs, self.ptrs, self.sfs, self.sf_ptrs = [], [], [], []
        for _ in range(2):
            buf = symm.empty((rows, n), dtype=torch.bfloat16 if payload == "bf16" else torch.uint8, device=dev)
            self.bufs.append(buf)
            self.ptrs.append([int(p) for p in symm.rendezvous(buf, self.group).buffer_ptrs])
            if payload == "mxfp8":
                sf = symm.empty((ops.sf_bytes(rows, n // 32),), dtype=torch.uint8, device=dev)
                self.sfs.append(sf)
                self.sf_ptrs.append([int(p) for p in symm.rendezvous(sf, self.group).buffer_ptrs])
        self._flag = torch.zeros(1, device=dev)
        self._turn = 0

    @property
    def buf(self) -> torch.Tensor:
        """The set the last call filled."""
        return self.bufs[self._turn ^ 1]

    def take(self) -> int:
        turn = self._turn
        self._turn ^= 1
        return turn

    def sync(self) -> None:
        """Stream-ordered rendezvous of the ranks: once it has run, every rank's stores have landed."""
        dist.all_reduce(self._flag, group=self.group)


def sharded_gemm_fused(a_shard: torch.Tensor, w: torch.Tensor, fmt: str, out: GatheredOutput):
    """`a_shard @ w.T` for this rank's rows of A (w is the (n, k) weight, replicated), quantized to
    `fmt` ("mxfp8", "nvfp4" or "fp8_e4m3" with per-row scales), with the output all-gather fused
    into the GEMM's epilogue.  Returns the gathered (world * m, n) bf16 matrix, or for an "mxfp8"
    payload the gathered (codes, scale factors); complete on return (this function runs the
    rendezvous) and valid until the call after the next one reuses the buffers."""
    from . import ops
    if a_shard.shape[0] != out.m or w.shape[0] != out.n:
        raise ValueError("shard / weight shape does not match the gathered output")
    turn = out.take()
    ptrs = out.ptrs[turn]
    if out.payload == "mxfp8":
        if fmt not in ("mxfp8", "mxfp8_e4m3"):
            raise ValueError("the MXFP8 payload is produced by the MXFP8 GEMM")
        ca, sfa = ops.quantize_mxfp8(a_shard, 1)
        cb, sfb = ops.quantize_mxfp8(w, 1)
        ops.gemm_mxfp8_allgather_mxfp8(ca, sfa, cb, sfb, ptrs, out.sf_ptrs[turn], out.rank, out.n, out.n)
        out.sync()
        return out.bufs[turn], out.sfs[turn]
    if fmt in ("mxfp8", "mxfp8_e4m3"):
        ca, sfa = ops.quantize_mxfp8(a_shard, 1)
        cb, sfb = ops.quantize_mxfp8(w, 1)
        ops.gemm_mxfp8_allgather(ca, sfa, cb, sfb, ptrs, out.rank, out.n, out.n)
    elif fmt in ("nvfp4", "fp4_nv"):
        pa, sfa, ta = ops.quantize_nvfp4(a_shard, 1)
        pb, sfb, tb = ops.quantize_nvfp4(w, 1)
        ops.gemm_nvfp4_allgather(pa, sfa, ta, pb, sfb, tb, ptrs, out.rank, out.n, out.n)
    elif fmt in ("fp8", "fp8_e4m3"):
        e4 = torch.float8_e4m3fn
        ca, sa = ops.quantize_fp8(a_shard, e4, 1)
        cb, sb = ops.quantize_fp8(w, e4, 1)
        ops.gemm_fp8_allgather(ca, e4, cb, e4, sa, sb, ptrs, out.rank, out.n, out.n)
    else:
        raise ValueError(f"unsupported format for the fused GEMM + all-gather: {fmt!r}")
    out.sync()
    return out.bufs[turn]


class ScatteredSum:
    """Staging for a GEMM whose (rows, cols) result is summed over the ranks and scattered by rows
    (reduce-scatter), as symmetric memory: rank g owns rows [g * rows / world, ...) and keeps one slot
    per sender; the senders' GEMM epilogues store their blocks of those rows straight into their slot
    over NVLink.  Two staging buffers alternate, so a rank that runs ahead writes the buffer its
    peers are not reading; one rendezvous per call orders everything else."""

    def __init__(self, rows: int, cols: int, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if rows % self.world or (rows // self.world) % 32 or cols % 8:
            raise ValueError("rows must split into multiples of 32 per rank and cols be a multiple of 8")
        self.rows, self.cols = rows, cols
        dev = torch.device("cuda", torch.cuda.current_device())
        self.bufs, self.ptrs = [], []
        for _ in range(2):
            buf = symm.empty((self.world, rows // self.world, cols), dtype=torch.bfloat16, device=dev)
            handle = symm.rendezvous(buf, self.group)
            self.bufs.append(buf)
            self.ptrs.append([int(p) for p in handle.buffer_ptrs])
        self._flag = torch.zeros(1, device=dev)
        self._turn = 0

    def sync(self) -> None:
        dist.all_reduce(self._flag, group=self.group)


def wgrad_reduce_scatter_fused(dy_shard: torch.Tensor, x_shard: torch.Tensor, out: ScatteredSum) -> torch.Tensor:
    """Data-parallel weight gradient of a linear layer in MXFP8: every rank holds its shard of the tokens
    (dy_shard (m, n) output gradients, x_shard (m, k) inputs, m % 32 == 0); returns this rank's rows
    [rank * n / world, ...) of dW = sum over ranks of dy_shard.T @ x_shard, bf16 (n / world, k).  The GEMM is the
    wgrad of QuantizedLinearFn (E5M2 gradients x E4M3 activations, blocks along the tokens,
    src/quant/linear.py:102-109); its epilogue does the scatter, a small kernel the sum."""
    from . import ops
    if dy_shard.shape[1] != out.rows or x_shard.shape[1] != out.cols or dy_shard.shape[0] != x_shard.shape[0]:
        raise ValueError("shards do not match the staged (n, k) result")
    gt, gtsf = ops.quantize_mxfp8(dy_shard, 0, torch.float8_e5m2)           # (n, m): blocks along the tokens
    xt, xtsf = ops.quantize_mxfp8(x_shard, 0, torch.float8_e4m3fn)          # (k, m)
    turn = out._turn
    out._turn ^= 1
    ops.gemm_mxfp8_scatter(gt, gtsf, xt, xtsf, out.ptrs[turn], out.rank, out.cols, out.cols, torch.float8_e5m2, torch.float8_e4m3fn)
    out.sync()
    return ops.sum_slots(out.bufs[turn])


class DataParallelGrad:
    """Sum of a linear layer's weight gradient over the ranks of a data-parallel group (the all-reduce DDP would do for
    the parameter), with the reduce-scatter half fused into the wgrad GEMM: ``wgrad`` runs the MXFP8 GEMM in scatter mode
    (every 32-row block of this rank's partial dW goes to this rank's slot in its owner's staging buffer over NVLink),
    rendezvous, each owner adds its slots in fp32 in rank order and rounds once, and an all-gather of the owners' shards
    gives every rank the full summed gradient - bit-identical on all ranks, and equal to adding the ranks' bf16 partials
    in fp32.  The reference is single-GPU: its wgrad is src/quant/linear.py:102-109 and nothing sums it."""

    def __init__(self, out_features: int, in_features: int, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.n, self.k = out_features, in_features
        self.fused = out_features % (32 * self.world) == 0 and in_features % 8 == 0
        self.stage = ScatteredSum(out_features, in_features, self.group) if self.fused else None

    def wgrad(self, gc, gsc, xc, xsc, fg, fa) -> torch.Tensor:
        """dW (n, k) bf16 summed over the ranks from this rank's transposed MXFP8 codes of the output gradient (n, m) and
        of the layer input (k, m)."""
        from . import ops
        if not self.fused:
            return self.reduce_small(ops.gemm_mxfp8(gc, gsc, xc, xsc, fg, fa))
        st = self.stage
        turn = st._turn
        st._turn ^= 1
        ops.gemm_mxfp8_scatter(gc, gsc, xc, xsc, st.ptrs[turn], st.rank, self.k, self.k, fg, fa)
        st.sync()
        shard = ops.sum_slots(st.bufs[turn])                                # this rank's rows of the sum
        full = torch.empty(self.n, self.k, dtype=torch.bfloat16, device=shard.device)
        dist.all_gather_into_tensor(full, shard, group=self.group)
        return full

    def reduce_small(self, t: torch.Tensor) -> torch.Tensor:
        """fp32 sum over the ranks of a gradient that has no fused form (a bias, or a weight of another format)."""
        acc = t.float().contiguous()
        dist.all_reduce(acc, group=self.group)
        return acc.to(t.dtype)


# ---- expert parallelism ---------------------------------------------------------------------

@dataclass
class DispatchState:
    send_order: torch.Tensor      # (n_pairs,) flat (token, slot) index of every sent row, in send order
    send_splits: list             # rows sent to each rank
    recv_splits: list             # rows received from each rank
    recv_expert: torch.Tensor     # (n_recv,) local expert id of every received row
    n_pairs: int


def ep_dispatch(x: torch.Tensor, top_indices: torch.Tensor, n_experts: int, group=None):
    """Send every routed (token, slot) pair's row to the rank that owns its expert.

    Experts are split in contiguous ranges of n_experts / world.  Rows leave sorted by (expert, token,
    slot) — the reference's stable expert order (src/layers/mlp.py:447-452) restricted to each
    destination — after a count exchange that tells every rank how many rows per local expert each
    peer sends.  Returns (received rows, DispatchState)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split evenly over {world} ranks")
    e_local = n_experts // world
    t, k = top_indices.shape
    flat_e = top_indices.reshape(-1)
    _, order = flat_e.sort(stable=True)
    counts = torch.bincount(flat_e, minlength=n_experts)                      # rows per global expert
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)                  # [src rank][local expert]
    send_splits = counts.view(world, e_local).sum(1).tolist()
    recv_mat = recv_counts.view(world, e_local)
    recv_splits = recv_mat.sum(1).tolist()
    rows = x[order // k]                                                      # expert-sorted rows
    recv = rows.new_empty(sum(recv_splits), x.shape[1])
    dist.all_to_all_single(recv, rows.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
    local_ids = torch.arange(e_local, device=x.device).repeat(world)
    recv_expert = torch.repeat_interleave(local_ids, recv_mat.reshape(-1))
    return recv, DispatchState(order, send_splits, recv_splits, recv_expert, t * k)


def ep_combine(y: torch.Tensor, state: DispatchState, top_weights: torch.Tensor, group=None) -> torch.Tensor:
    """Return every processed row to its sender and reduce the k rows of a token with its routing
    weights (fp32 accumulation, one rounding — as b200q_moe_unpermute does)."""
    back = y.new_empty(state.n_pairs, y.shape[1])
    dist.all_to_all_single(back, y.contiguous(), output_split_sizes=state.send_splits, input_split_sizes=state.recv_splits,
                           group=group)
    t, k = top_weights.shape
    per_pair = torch.empty_like(back)
    per_pair[state.send_order] = back                                          # undo the expert sort
    w = top_weights.reshape(t, k, 1).float()
    return (per_pair.view(t, k, -1).float() * w).sum(1).to(y.dtype)


class FusedExpertParallel:
    """Expert-parallel MoE inside one NVLink domain with the exchange done by the kernels themselves: the dispatch
    stores each routed row straight into the buffer of the rank that owns its expert, the combine loads the expert outputs
    in place from their owners.  Per call there is ONE collective, an all-gather of the per-expert counts (E integers per
    rank); the phases are ordered by a flag barrier in peer-mapped memory (b200q_peer_barrier: bounded waits, no NCCL),
    and every index table - where my rows start at each owner, the segment ends of my own experts, owner and row of each
    routed pair - comes from one kernel (b200q_moe_ep_index).

    ``forward`` is the gradient-free path (MXFP8 codes + scale factors on the wire, SwiGLU in the first GEMM's epilogue).
    ``train`` is differentiable: bf16 rows on the wire (an owner needs both MXFP8 directions of what it receives, and the
    transposed one cannot be made by the senders), the owner's four backward GEMMs in MXFP8 as on one GPU, the output
    gradient scattered to the owners and the input gradient combined back the same way.

    Buffers are symmetric memory sized for `capacity_rows` received rows per rank (default: every routed row of every
    rank, which cannot overflow; a smaller capacity is checked on the host every call).  One instance serves one layer:
    ``train`` keeps the expert outputs in its buffer until the matching backward has run.  Results equal the single-GPU
    block on the concatenated tokens bit for bit when the ranks hold consecutive token ranges (the routing weights'
    gradient, a dot product summed in another order, within fp32 rounding)."""

    def __init__(self, tokens_per_rank: int, top_k: int, d_model: int, n_experts: int, group=None, capacity_rows: int | None = None,
                 training: bool = False):
        import torch.distributed._symmetric_memory as symm
        from . import ops
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if n_experts % self.world or d_model % 128:
            raise ValueError("experts must split evenly over the ranks and d_model must be a multiple of 128")
        self.e, self.e_local, self.d, self.k, self.t = n_experts, n_experts // self.world, d_model, top_k, tokens_per_rank
        rows = capacity_rows if capacity_rows is not None else self.world * tokens_per_rank * top_k
        self.rows, self.check_capacity = rows, capacity_rows is not None       # the default capacity cannot overflow
        self.cap = ops.moe_padded_rows(rows, self.e_local)
        dev = torch.device("cuda", torch.cuda.current_device())
        self._handles = []

        def shared(shape, dtype):
            buf = symm.empty(shape, dtype=dtype, device=dev)
            h = symm.rendezvous(buf, self.group)
            self._handles.append(h)
            return buf, [int(p) for p in h.buffer_ptrs]

        self.codes, self.codes_ptrs = shared((self.cap, d_model), torch.uint8)
        self.sf, self.sf_ptrs = shared((ops.sf_bytes(self.cap, d_model // 32),), torch.uint8)
        self.y, self.y_ptrs = shared((self.cap, d_model), torch.bfloat16)
        self.flags, self.flag_ptrs = shared((8,), torch.int32)
        self.training = training
        if training:
            self.xin, self.xin_ptrs = shared((self.cap, d_model), torch.bfloat16)     # received rows
            self.dy, self.dy_ptrs = shared((self.cap, d_model), torch.bfloat16)       # received output gradients
            self.da, self.da_ptrs = shared((self.cap, d_model), torch.bfloat16)       # input gradients of my experts' rows
        self.flags.zero_()
        self._epoch = 0
        self._ones = None
        self._ws = None
        torch.cuda.synchronize()
        dist.barrier(group=self.group)                       # every rank's flags are zero before anyone signals

    def _rendezvous(self):
        """Stream-ordered: the kernels before it have stored, the kernels after it start once every rank has arrived."""
        from . import ops
        self._epoch += 1
        ops.peer_barrier(self.flag_ptrs, self.rank, self._epoch)

    def _tables(self, top_indices: torch.Tensor):
        from . import ops
        plan = ops.moe_permute_plan(top_indices, self.e)                                       # my rows in my own stable expert order
        all_offs = torch.empty(self.world, self.e, dtype=torch.int32, device=top_indices.device)
        dist.all_gather_into_tensor(all_offs, plan.offs, group=self.group)                      # [sender][global expert], cumulative
        row_base, own_offs, pair_peer, pair_row = ops.moe_ep_index(all_offs, self.rank, top_indices, plan)
        if self.check_capacity:                                                                 # host sync
            counts = torch.diff(all_offs, dim=1, prepend=all_offs.new_zeros(self.world, 1)).sum(0)
            need = ((counts + 127) // 128 * 128).view(self.world, self.e_local).sum(1).max()
            if int(need) > self.cap or int(own_offs[-1]) > self.rows:
                raise RuntimeError("received rows exceed the capacity of the expert-parallel buffers")
        own = ops.moe_pad_plan(own_offs, self.rows)                                             # segment table of the experts I own
        return plan, own, row_base, pair_peer, pair_row

    def forward(self, x: torch.Tensor, top_indices: torch.Tensor, top_weights: torch.Tensor, w_in_local: torch.Tensor,
                w_down_local: torch.Tensor) -> torch.Tensor:
        from . import ops
        from .layers.mlp import _grouped_ffn_padded, silu_glu
        plan, own, row_base, pair_peer, pair_row = self._tables(top_indices)
        inter = w_down_local.shape[2]
        if w_in_local.shape[1] == 2 * inter and inter % 64 == 0 and own.padded_rows == self.cap:
            # everything after the tables as one library call on a standing workspace
            from .layers.mlp import _expert_weight_copies
            w1c, w1s = _expert_weight_copies(w_in_local if w_in_local.dtype == torch.bfloat16 else w_in_local.to(torch.bfloat16), "glu")
            w2c, w2s = _expert_weight_copies(w_down_local if w_down_local.dtype == torch.bfloat16 else w_down_local.to(torch.bfloat16), "rows")
            need = ops.moe_ep_forward_workspace_bytes(self.cap, inter)
            if self._ws is None or self._ws.numel() < need:
                self._ws = torch.empty(need, dtype=torch.uint8, device=x.device)
            out = ops.moe_ep_forward(x.to(torch.bfloat16), top_weights, plan, own, row_base, pair_peer, pair_row, self.e_local, self.rank,
                                     self._epoch, self.codes_ptrs, self.sf_ptrs, self.y_ptrs, self.flag_ptrs, w1c, w1s, w2c, w2s, inter,
                                     self._ws)
            self._epoch += 3
            return out.to(x.dtype)
        ops.moe_zero_pad_rows(own, self.d, self.codes, self.sf)
        ops.moe_dispatch_peers(x.to(torch.bfloat16), plan, row_base, self.e_local, self.codes_ptrs, self.sf_ptrs)
        self._rendezvous()
        _grouped_ffn_padded(self.codes, self.sf, own, w_in_local.to(torch.bfloat16), w_down_local.to(torch.bfloat16), silu_glu, True,
                            out=self.y)                        # the second GEMM writes where the peers will read
        self._rendezvous()
        out = ops.moe_combine_peers(self.y_ptrs, self.d, top_weights, pair_peer, pair_row, self.d)
        self._rendezvous()                                   # nobody overwrites y or the codes while a peer still reads them
        return out.to(x.dtype)

    def train(self, x: torch.Tensor, top_indices: torch.Tensor, top_weights: torch.Tensor, w_in_local: torch.Tensor,
              w_down_local: torch.Tensor) -> torch.Tensor:
        """Differentiable forward: gradients flow to x, top_weights and this rank's expert weights."""
        if not self.training:
            raise RuntimeError("construct FusedExpertParallel(..., training=True) for the differentiable path")
        return _FusedEPTrainFn.apply(x, top_weights, w_in_local, w_down_local, self, top_indices)


class _FusedEPTrainFn(torch.autograd.Function):
    """Forward and backward of the expert-parallel block (SwiGLU experts without biases): the single-GPU expert path
    (layers/mlp.py::_ExpertFFN) with its gather and unpermute replaced by peer scatters and combines."""

    @staticmethod
    def forward(ctx, x, top_w, w_in, w_down, ep, top_indices):
        from . import ops
        from .layers.mlp import _expert_weight_copies
        E4, SWZ = ops.E4M3, ops.SF_SWIZZLED
        d, k = ep.d, ep.k
        n1 = w_in.shape[1]
        inter = n1 // 2
        if d % 128 or n1 % 128 or inter % 32:
            raise NotImplementedError("d_model and 2 * intermediate_size must be multiples of 128, intermediate_size of 32")
        plan, own, row_base, pair_peer, pair_row = ep._tables(top_indices)
        nt = own.num_tiles
        ops.moe_zero_pad_rows_bf16(own, ep.xin)
        ops.moe_scatter_rows_peers(x.to(torch.bfloat16), None, pair_peer, pair_row, k, ep.xin_ptrs, d)      # dispatch: bf16 rows
        ep._rendezvous()
        ar, asr, ac, asc = ops.quantize_mxfp8_dual(ep.xin, E4, SWZ, num_tiles=nt)
        w1r, w1sr, w1c, w1sc = _expert_weight_copies(w_in, "dual")
        w2r, w2sr, w2c, w2sc = _expert_weight_copies(w_down, "dual")
        g = ops.grouped_gemm_mxfp8(ar, asr, w1r, w1sr, own, n1)                                  # (cap, 2I) bf16, kept for backward
        if inter % 128 == 0:
            hr, hsr, hc, hsc = ops.swiglu_quantize_dual(g, E4, num_tiles=nt)
        else:
            hr, hsr, hc, hsc = ops.quantize_mxfp8_dual(ops.swiglu(g, False), E4, SWZ, num_tiles=nt)
        ops.grouped_gemm_mxfp8(hr, hsr, w2r, w2sr, own, d, out=ep.y)                             # where the peers read
        ep._rendezvous()
        out = ops.moe_combine_peers(ep.y_ptrs, d, top_w, pair_peer, pair_row, d)
        ep._rendezvous()
        ctx.save_for_backward(top_w, ac, asc, g, hc, hsc, w1c, w1sc, w2c, w2sc, pair_peer, pair_row, own.offs, own.padded_offs,
                              own.src_of_row, own.tile_expert, own.num_tiles)
        ctx.ep, ctx.own_rows, ctx.inter = ep, own.padded_rows, inter
        ctx.dtypes = (x.dtype, top_w.dtype, w_in.dtype, w_down.dtype)
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        from . import ops
        (top_w, ac, asc, g, hc, hsc, w1c, w1sc, w2c, w2sc, pair_peer, pair_row, o_offs, o_poffs, o_src, o_tile, o_nt) = ctx.saved_tensors
        ep, inter = ctx.ep, ctx.inter
        E4, E5, SWZ = ops.E4M3, ops.E5M2, ops.SF_SWIZZLED
        d, k = ep.d, ep.k
        own = ops.MoEPlan()
        own.offs, own.padded_offs, own.src_of_row, own.tile_expert, own.num_tiles = o_offs, o_poffs, o_src, o_tile, o_nt
        own.row_of, own.padded_rows, own.n_experts = None, ctx.own_rows, ep.e_local
        dout = dout.reshape(-1, d).to(torch.bfloat16).contiguous()
        dw = ops.moe_pair_dots_peers(dout, ep.y_ptrs, d, pair_peer, pair_row, k)                 # <dout, y>: y still in the owners' buffers
        ops.moe_zero_pad_rows_bf16(own, ep.dy)
        ops.moe_scatter_rows_peers(dout, top_w, pair_peer, pair_row, k, ep.dy_ptrs, d)           # dy = w * dout, to the owners
        ep._rendezvous()
        dyr, dysr, dyc, dysc = ops.quantize_mxfp8_dual(ep.dy, E5, SWZ, num_tiles=o_nt)
        dh = ops.grouped_gemm_mxfp8_dgrad(dyr, dysr, w2c, w2sc, own, inter, E5, E4)              # (cap, I)
        dw2 = ops.grouped_gemm_mxfp8_wgrad(dyc, dysc, hc, hsc, own, E5, E4)                      # (E_local, D, I)
        dgr, dgsr, dgc, dgsc = ops.swiglu_backward_quantize_dual(g, dh, E5, num_tiles=o_nt)
        ops.grouped_gemm_mxfp8_dgrad(dgr, dgsr, w1c, w1sc, own, d, E5, E4, out=ep.da)            # where the peers read
        dw1 = ops.grouped_gemm_mxfp8_wgrad(dgc, dgsc, ac, asc, own, E5, E4)                      # (E_local, 2I, D)
        ep._rendezvous()
        if ep._ones is None or ep._ones.shape != top_w.shape:
            ep._ones = torch.ones(top_w.shape, dtype=torch.bfloat16, device=dout.device)
        dx = ops.moe_combine_peers(ep.da_ptrs, d, ep._ones, pair_peer, pair_row, d)              # sum over the k slots
        ep._rendezvous()
        xd, twd, w1d, w2d = ctx.dtypes
        return dx.to(xd), dw.to(twd), dw1.to(w1d), dw2.to(w2d), None, None


def expert_ffn_local(rows: torch.Tensor, expert_ids: torch.Tensor, w_in: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Gated-SwiGLU expert FFN for rows in ARBITRARY order with their local expert ids, on the
    MXFP8 kernels: local permute plan, fused gather+quantize, two grouped GEMMs with the fused
    SwiGLU between them, rows returned in the input order."""
    from . import ops
    from .layers.mlp import _grouped_ffn_padded, silu_glu
    if rows.shape[0] == 0:
        return rows.new_empty(0, w_down.shape[1])
    plan = ops.moe_permute_plan(expert_ids.view(-1, 1), w_in.shape[0])
    a, sfa = ops.moe_gather(rows, plan, True)
    y = _grouped_ffn_padded(a, sfa, plan, w_in, w_down, silu_glu, True)
    return y[plan.row_of.long()]


def expert_parallel_moe(x: torch.Tensor, top_indices: torch.Tensor, top_weights: torch.Tensor, w_in_local: torch.Tensor,
                        w_down_local: torch.Tensor, n_experts: int, group=None, ffn: Callable = expert_ffn_local) -> torch.Tensor:
    """Expert-parallel MoE forward for this rank's tokens: dispatch all-to-all, local expert FFN
    on this rank's experts (`w_*_local` are its (E/world, out, in) slices), combine all-to-all,
    weighted reduction.  Equals the single-GPU block on the concatenated tokens."""
    recv, state = ep_dispatch(x, top_indices, n_experts, group)
    y = ffn(recv, state.recv_expert, w_in_local, w_down_local)
    return ep_combine(y, state, top_weights, group)
