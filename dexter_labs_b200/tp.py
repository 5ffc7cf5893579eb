"""Tensor-parallel sharding of packed weights and the linear-layer set built on it.

The reference is a single-device engine (its README states multi-GPU is out of
scope), so nothing here has a counterpart there; the unsharded reference result
is the oracle.  What it has to respect is the reference's packed layout
(``python/dexter/quant.py:62-133``):

* column-parallel (QKV, cross Q/K/V, FFN-up): every output column owns one
  column of ``qweight`` / ``scales`` / ``zeros`` / ``bias``, so a shard is a plain
  slice along N -- bit-identical to quantising the sliced weight.
* row-parallel (O, FFN-down): a packed int4 byte row carries logical rows ``i``
  and ``i + K/2``, so slicing packed rows would hand a rank two disjoint K ranges.
  Instead the weight is cut in the LOGICAL domain on whole quantisation groups
  (group statistics are per group and column, so this is again bit-identical to
  quantising the slice) and every shard is re-packed split-half on its own.
  Each rank then multiplies its contiguous slice of the activation columns and
  the partial products are summed across ranks; the bias rides on rank 0 only.

``LayerSet`` strings the ten linears of a DiT block (self q/k/v/o, cross
q/k/v/o, FFN up/down; shapes from ``python/dexter/models/dreamzero/config.py``
and ``model.py:148-151,204-207,260-261``) into column->row pairs with one
reduce-scatter + all-gather (or all-reduce) after every row-parallel linear.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from .quant import QuantizedWeight, pack_nibbles, quantize

__all__ = ["group_bounds", "split_columns", "split_rows", "concat_columns", "ShardedLinear", "LayerSet", "PRESETS",
           "unpack_nibbles"]

# name -> (dim, ffn_dim, blocks); python/dexter/models/dreamzero/config.py:182-219
PRESETS: Dict[str, Tuple[int, int, int]] = {"5b": (3072, 14336, 30), "14b": (5120, 13824, 40)}

GemmFn = Callable[[torch.Tensor, QuantizedWeight], torch.Tensor]


def unpack_nibbles(qweight: torch.Tensor) -> torch.Tensor:
    """``[K/2, N]`` packed bytes -> ``[K, N]`` values 0..15 (low nibbles first)."""
    return torch.cat((qweight & 0x0F, (qweight >> 4) & 0x0F), dim=0)


def group_bounds(num_groups: int, rank: int, world: int) -> Tuple[int, int]:
    """Whole groups ``[g0, g1)`` owned by ``rank``; sizes differ by at most one group."""
    base, extra = divmod(num_groups, world)
    g0 = rank * base + min(rank, extra)
    return g0, g0 + base + (1 if rank < extra else 0)


def split_columns(qw: QuantizedWeight, rank: int, world: int) -> QuantizedWeight:
    """Column-parallel shard: columns ``[rank*N/world, (rank+1)*N/world)`` of every tensor."""
    k, n = qw.shape
    if n % world:
        raise ValueError(f"N={n} does not split into {world} column shards")
    n0, n1 = rank * n // world, (rank + 1) * n // world

    def cut(t):
        return None if t is None else t[..., n0:n1].contiguous()

    return QuantizedWeight(cut(qw.qweight), cut(qw.scales), cut(qw.zeros), cut(qw.bias),
                           qw.group_size, qw.bits, (k, n1 - n0))


def split_rows(qw: QuantizedWeight, rank: int, world: int) -> Tuple[QuantizedWeight, Tuple[int, int]]:
    """Row-parallel shard on whole groups, re-packed; returns it with its K range ``(k0, k1)``."""
    k, n = qw.shape
    g = qw.group_size
    if k // g < world:
        raise ValueError(f"K={k} has {k // g} group(s) of {g}: fewer than the {world} ranks")
    g0, g1 = group_bounds(k // g, rank, world)
    k0, k1 = g0 * g, g1 * g
    if qw.bits == 4:
        logical = unpack_nibbles(qw.qweight)[k0:k1]
        if (k1 - k0) % 2:
            raise ValueError("an int4 shard needs an even number of rows")
        packed = pack_nibbles(logical)
    else:
        packed = qw.qweight[k0:k1].contiguous()
    shard = QuantizedWeight(packed, qw.scales[g0:g1].contiguous(),
                            None if qw.zeros is None else qw.zeros[g0:g1].contiguous(),
                            qw.bias if rank == 0 else None, g, qw.bits, (k1 - k0, n))
    return shard, (k0, k1)


def concat_columns(parts: List[QuantizedWeight]) -> QuantizedWeight:
    """N-concatenation of packed weights that share K, group size and bit width.

    Scales, zero points and bias are per column, so one GEMM on the concatenation does
    the same arithmetic per column as separate GEMMs on the parts (bit-identical for a
    fixed K-summation order; this is how separate q/k/v linears become one
    ``dim -> 3*dim`` launch).
    """
    first = parts[0]
    if any(p.shape[0] != first.shape[0] or p.bits != first.bits or p.group_size != first.group_size
           or (p.zeros is None) != (first.zeros is None) or (p.bias is None) != (first.bias is None)
           for p in parts):
        raise ValueError("only weights with the same K, bits, group size and zero/bias presence concatenate")

    def cat(ts):
        return None if ts[0] is None else torch.cat(ts, dim=-1).contiguous()

    return QuantizedWeight(cat([p.qweight for p in parts]), cat([p.scales for p in parts]),
                           cat([p.zeros for p in parts]), cat([p.bias for p in parts]),
                           first.group_size, first.bits, (first.shape[0], sum(p.shape[1] for p in parts)))


@dataclass
class ShardedLinear:
    """One linear of the set on one rank."""

    name: str
    kind: str  # "column" | "row"
    weight: QuantizedWeight
    k_range: Tuple[int, int]  # activation columns this rank consumes
    full_shape: Tuple[int, int]  # unsharded (K, N)
    layout: str = "dexter"       # "b200" once the packed int4 bytes went through ops.relayout_w4
    full_bias: Optional[torch.Tensor] = None  # row-parallel: the linear's bias on EVERY rank

    @property
    def weight_bytes(self) -> int:
        return self.weight.nbytes

    def flops(self, m: int) -> int:
        k, n = self.weight.shape
        return 2 * m * k * n


def _default_gemm(x: torch.Tensor, w: QuantizedWeight, max_ctas: int = 0, *, layout: str = "dexter",
                  reduce=None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    from . import ops

    bias = w.bias if bias is None else bias
    if w.bits == 4:
        return ops.w4a16(x, w.qweight, w.scales, w.zeros, bias, w.group_size, max_ctas=max_ctas,
                         layout=layout, reduce=reduce)
    return ops.w8a16(x, w.qweight, w.scales, w.zeros, bias, w.group_size, max_ctas=max_ctas, reduce=reduce)


# (name, input, kind): the ten linears of one DiT block in execution order
_BLOCK_PLAN = (
    ("self_q", "dim", "column"), ("self_k", "dim", "column"), ("self_v", "dim", "column"),
    ("self_o", "dim", "row"),
    ("cross_q", "dim", "column"), ("cross_k", "dim", "column"), ("cross_v", "dim", "column"),
    ("cross_o", "dim", "row"),
    ("ffn_up", "dim", "column"), ("ffn_down", "ffn", "row"),
)


@dataclass
class LayerSet:
    """The quantised linears of ``blocks`` DiT blocks, sharded for one rank.

    ``forward`` runs them as column->row pairs.  There is no attention, norm or
    activation function between them (those are other ops of the reference, not part
    of this path): the column-parallel output that would feed attention goes
    straight into the row-parallel projection, which keeps every GEMM's shape,
    bytes and flops exactly those of the model.
    """

    dim: int
    ffn_dim: int
    blocks: int
    rank: int = 0
    world: int = 1
    bits: int = 4
    group_size: int = 128
    collective: str = "rs_ag"  # "rs_ag" | "all_reduce" (NCCL) | "peer" (own all-reduce kernel over peer
                               # memory) | "fused" (the sum is part of the row-parallel GEMM's launch)
    fuse_qkv: bool = False     # one launch for self q,k,v and one for cross k,v (N-concatenation)
    concurrent: bool = False   # independent linears of a block on parallel CUDA streams
    layers: List[List[ShardedLinear]] = field(default_factory=list)
    gemm: GemmFn = _default_gemm
    process_group: Optional[object] = None
    _pad: Dict[Tuple[int, int], torch.Tensor] = field(default_factory=dict)
    _side: Optional[list] = None
    _sms: int = 0
    _peer: Optional[object] = None  # ops.PeerAllReduce, see enable_peer_reduce
    _fused: Optional[object] = None  # ops.FusedReduce, see enable_fused_reduce
    _plain: Dict[int, QuantizedWeight] = field(default_factory=dict)  # see _g

    def enable_peer_reduce(self, tokens: int, device) -> bool:
        """Set up the peer-memory all-reduce for outputs of up to ``tokens x dim`` bf16.

        A collective: every rank calls it at the same point.  Returns False (and the set
        keeps using NCCL's all-reduce) when peer-mapped memory cannot be set up on any rank.
        """
        import torch.distributed as dist

        from . import ops

        group = self.process_group if self.process_group is not None else dist.group.WORLD
        peer, ok = None, 1
        try:
            peer = ops.PeerAllReduce(group, tokens * self.dim, torch.device(device))
        except Exception as exc:  # noqa: BLE001 - reported below, every rank must agree
            ok = 0
            self._peer_error = repr(exc)
        flag = torch.tensor([ok], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 1:
            self._peer = peer
            self.collective = "peer"
            return True
        self._peer = None
        self.collective = "all_reduce"
        return False

    def enable_fused_reduce(self, tokens: int, device) -> bool:
        """Set up the sum over ranks INSIDE the row-parallel GEMMs (``collective="fused"``) for
        outputs of up to ``tokens x dim`` bf16, at most 128 tokens.  A collective: every rank
        calls it at the same point.  Returns False (nothing changes) when peer-mapped memory
        cannot be set up on every rank."""
        import torch.distributed as dist

        from . import ops

        group = self.process_group if self.process_group is not None else dist.group.WORLD
        ctx, ok = None, 1
        try:
            if tokens > 128:
                raise ValueError("the fused sum over ranks takes at most 128 tokens")
            ctx = ops.FusedReduce(group, tokens * self.dim, torch.device(device))
        except Exception as exc:  # noqa: BLE001 - reported below, every rank must agree
            ok = 0
            self._peer_error = repr(exc)
        flag = torch.tensor([ok], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 1:
            self._fused = ctx
            self.collective = "fused"
            return True
        return False

    def relayout_(self) -> "LayerSet":
        """Load-time repack of every int4 weight of the set for the tensor-core kernel, in
        place (``ops.relayout_w4``); shapes that kernel does not take keep the reference layout."""
        from . import ops

        for row in self.layers:
            for l in row:
                q = l.weight.qweight
                if (l.layout == "dexter" and l.weight.bits == 4 and q.is_cuda and q.shape[0] % 64 == 0
                        and q.shape[1] % 16 == 0 and l.weight.group_size % 64 == 0 and q.is_contiguous()):
                    ops.relayout_w4(q, out=q)
                    l.layout = "b200"
        return self

    # ------------------------------------------------------------------ build
    @classmethod
    def build(cls, preset: str, *, blocks: Optional[int] = None, rank: int = 0, world: int = 1,
              bits: int = 4, group_size: int = 128, symmetric: bool = True, bias: bool = True,
              device="cuda", seed: int = 0, collective: str = "rs_ag", gemm: GemmFn = _default_gemm,
              process_group=None, weight_std: float = 0.02, fuse_qkv: bool = False,
              concurrent: bool = False, relayout: bool = True) -> "LayerSet":
        dim, ffn, nblocks = PRESETS[preset]
        nblocks = blocks if blocks is not None else nblocks
        self = cls(dim=dim, ffn_dim=ffn, blocks=nblocks, rank=rank, world=world, bits=bits,
                   group_size=group_size, collective=collective, fuse_qkv=fuse_qkv,
                   concurrent=concurrent, layers=[], gemm=gemm, process_group=process_group)
        for blk in range(nblocks):
            row: List[ShardedLinear] = []
            for idx, (name, src, kind) in enumerate(_BLOCK_PLAN):
                k = dim if src == "dim" else ffn
                n = ffn if name == "ffn_up" else dim
                gen = torch.Generator(device="cpu").manual_seed(seed + 1000 * blk + idx)
                w = (torch.randn(n, k, generator=gen) * weight_std).to(torch.bfloat16).to(device)
                b = (torch.randn(n, generator=gen) * 0.1).to(torch.bfloat16).to(device) if bias else None
                g = group_size if group_size > 0 else k
                full = quantize(w, bits=bits, group_size=g, bias=b, symmetric=symmetric)
                row.append(self.shard(name, kind, full))
                del w, full
            if fuse_qkv:
                row = self._fuse(row)
            self.layers.append(row)
        if relayout and gemm is _default_gemm and str(device).startswith("cuda"):
            self.relayout_()
        return self

    @staticmethod
    def _fuse(row: List[ShardedLinear]) -> List[ShardedLinear]:
        """Replace (self q,k,v) and (cross k,v) by their per-rank N-concatenations."""
        by = {l.name: l for l in row}
        out: List[ShardedLinear] = []
        for name in ("self_qkv", "self_o", "cross_q", "cross_kv", "cross_o", "ffn_up", "ffn_down"):
            if name in by:
                out.append(by[name])
                continue
            parts = [by[f"self_{c}"] for c in "qkv"] if name == "self_qkv" else [by["cross_k"], by["cross_v"]]
            fused = concat_columns([p.weight for p in parts])
            k = parts[0].full_shape[0]
            if len({p.layout for p in parts}) != 1:
                raise ValueError("only weights in the same layout concatenate")
            out.append(ShardedLinear(name, "column", fused, (0, k),
                                     (k, sum(p.full_shape[1] for p in parts)), layout=parts[0].layout))
        return out

    def shard(self, name: str, kind: str, full: QuantizedWeight) -> ShardedLinear:
        k, n = full.shape
        if self.world == 1:
            return ShardedLinear(name, kind, full, (0, k), (k, n))
        if kind == "column":
            return ShardedLinear(name, kind, split_columns(full, self.rank, self.world), (0, k), (k, n))
        part, k_range = split_rows(full, self.rank, self.world)
        return ShardedLinear(name, kind, part, k_range, (k, n), full_bias=full.bias)

    # ------------------------------------------------------------------ stats
    @property
    def num_gemms(self) -> int:
        """Kernel launches per pass (7 per block when q/k/v are fused, else 10)."""
        return sum(len(r) for r in self.layers)

    @property
    def num_linears(self) -> int:
        """Linears of the model computed per pass (10 per block either way)."""
        return len(_BLOCK_PLAN) * self.blocks

    @property
    def weight_bytes(self) -> int:
        return sum(l.weight_bytes for r in self.layers for l in r)

    def flops(self, m: int) -> int:
        return sum(l.flops(m) for r in self.layers for l in r)

    # ---------------------------------------------------------------- forward
    def _g(self, x: torch.Tensor, layer: ShardedLinear, max_ctas: int = 0) -> torch.Tensor:
        """One linear of the set on this rank (a partial product for a row-parallel one)."""
        if self.gemm is _default_gemm:
            return _default_gemm(x, layer.weight, max_ctas, layout=layer.layout)
        w = layer.weight
        if layer.layout != "dexter":
            # a caller-supplied GEMM (the CPU oracle in tests) reads the reference layout
            w = self._plain.get(id(layer))
            if w is None:
                from . import ops

                q = ops.relayout_w4(layer.weight.qweight, inverse=True)
                w = QuantizedWeight(q, layer.weight.scales, layer.weight.zeros, layer.weight.bias,
                                    layer.weight.group_size, layer.weight.bits, layer.weight.shape)
                self._plain[id(layer)] = w
        return self.gemm(x, w)

    def _row(self, col_out: torch.Tensor, layer: ShardedLinear) -> torch.Tensor:
        """A row-parallel linear including the sum over ranks: one launch when the sum is fused
        into the GEMM, else the GEMM followed by the collective."""
        xin = self._row_input(col_out, layer)
        if (self.world > 1 and self.collective == "fused" and self._fused is not None
                and self.gemm is _default_gemm and xin.shape[0] <= 128
                and xin.shape[0] * layer.full_shape[1] <= self._fused.capacity):
            return _default_gemm(xin, layer.weight, 0, layout=layer.layout, reduce=self._fused,
                                 bias=layer.full_bias)
        return self._reduce(self._g(xin, layer))

    def _reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum the row-parallel partial products over ranks; every rank gets the full result."""
        if self.world == 1:
            return partial
        import torch.distributed as dist

        if self.collective == "peer":
            # one kernel over NVLink peer memory for the small messages of the few-token
            # regime; anything larger goes to NCCL
            nbytes = partial.numel() * partial.element_size()
            if self._peer is not None and nbytes <= self._peer.MAX_BYTES and partial.numel() % 8 == 0 \
                    and partial.numel() <= self._peer.capacity:
                return self._peer(partial.contiguous())
            dist.all_reduce(partial, group=self.process_group)
            return partial
        if self.collective == "all_reduce":
            dist.all_reduce(partial, group=self.process_group)
            return partial
        m, n = partial.shape
        rows = -(-m // self.world)  # token rows per rank, padded so the scatter is even
        key = (rows * self.world, n)
        buf = self._pad.get(key)
        if buf is None or buf.device != partial.device:
            buf = torch.zeros(key, dtype=partial.dtype, device=partial.device)
            self._pad[key] = buf
        buf[:m].copy_(partial)
        mine = torch.empty((rows, n), dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(mine, buf, group=self.process_group)
        out = torch.empty_like(buf)
        dist.all_gather_into_tensor(out, mine, group=self.process_group)
        return out[:m]

    def _local_cols(self, full_cols: int) -> Tuple[int, int]:
        return self.rank * full_cols // self.world, (self.rank + 1) * full_cols // self.world

    def _block_forward_concurrent(self, blk: int, x: torch.Tensor, ctx: torch.Tensor) -> torch.Tensor:
        """Same linears and data dependencies as :meth:`block_forward`, but the ones that do
        not depend on each other run side by side: self q, k, v and cross k, v (which only
        need the block input and the context) start together on five streams, each capped
        to a fifth of the SMs; o waits for q, k, v; cross o waits for cross q, k, v.  Under
        CUDA-graph capture this becomes a fork/join graph."""
        L = {l.name: l for l in self.layers[blk]}
        g = self._g
        cur = torch.cuda.current_stream()
        if self._side is None:
            self._side = [torch.cuda.Stream() for _ in range(4)]
            self._sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        side = self._side
        if self.world > 1:
            return self._block_forward_overlapped(L, x, ctx)
        share = max(self._sms // 5, 1)
        for s in side:
            s.wait_stream(cur)
        outs = {}
        for s, (name, inp) in zip(side, (("self_q", x), ("self_k", x), ("cross_k", ctx), ("cross_v", ctx))):
            with torch.cuda.stream(s):
                outs[name] = g(inp, L[name], share)
        v = g(x, L["self_v"], share)
        cur.wait_stream(side[0])
        cur.wait_stream(side[1])
        x = self._row(v, L["self_o"])
        g(x, L["cross_q"])
        cur.wait_stream(side[2])
        cur.wait_stream(side[3])
        x = self._row(outs["cross_v"], L["cross_o"])
        h = g(x, L["ffn_up"])
        x = self._row(h, L["ffn_down"])
        return x

    def _block_forward_overlapped(self, L, x: torch.Tensor, ctx: torch.Tensor) -> torch.Tensor:
        """Schedule for more than one rank: the collective after self o is the place where the
        GPU would otherwise wait for NVLink, so cross k and cross v (which only need the
        context) are held back until self o's GEMM has been issued and then run on two side
        streams while that collective is in flight on the main stream."""
        g = self._g
        cur = torch.cuda.current_stream()
        side = self._side
        third = max(self._sms // 3, 1)
        half = max(self._sms // 2, 1)
        for s in side[:2]:
            s.wait_stream(cur)
        for s, name in zip(side[:2], ("self_q", "self_k")):
            with torch.cuda.stream(s):
                g(x, L[name], third)
        v = g(x, L["self_v"], third)
        cur.wait_stream(side[0])
        cur.wait_stream(side[1])
        outs = {}
        if self.collective == "fused":
            # the sum is inside self o's launch: fork before it, so cross k and cross v run
            # beside it and fill the SMs while it waits for the other ranks
            for s in side[2:]:
                s.wait_stream(cur)
            x = self._row(v, L["self_o"])
            for s, name in zip(side[2:], ("cross_k", "cross_v")):
                with torch.cuda.stream(s):
                    outs[name] = g(ctx, L[name], half)
        else:
            partial = g(self._row_input(v, L["self_o"]), L["self_o"])
            for s, name in zip(side[2:], ("cross_k", "cross_v")):
                s.wait_stream(cur)  # after self o's GEMM, alongside its collective
                with torch.cuda.stream(s):
                    outs[name] = g(ctx, L[name], half)
            x = self._reduce(partial)
        g(x, L["cross_q"])
        cur.wait_stream(side[2])
        cur.wait_stream(side[3])
        x = self._row(outs["cross_v"], L["cross_o"])
        h = g(x, L["ffn_up"])
        x = self._row(h, L["ffn_down"])
        return x

    def _block_forward_fused_overlapped(self, blk: int, x: torch.Tensor, ctx: torch.Tensor) -> torch.Tensor:
        """q/k/v fused (seven launches per block) with the fused cross k/v launch, which only
        needs the context, on a side stream.  One rank: it starts with the block, next to
        self q/k/v, each of the two capped to its share of the SMs.  More ranks: it is held
        back until self o's GEMM has been issued and runs while that GEMM's collective is in
        flight on the main stream."""
        L = {l.name: l for l in self.layers[blk]}
        g = self._g
        cur = torch.cuda.current_stream()
        if self._side is None:
            self._side = [torch.cuda.Stream() for _ in range(4)]
            self._sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        side = self._side[0]
        if self.world == 1:
            kv_tiles = -(-L["cross_kv"].weight.qweight.shape[1] // 128)
            kv_share = max(min(kv_tiles, self._sms // 3), 1)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                kv = g(ctx, L["cross_kv"], kv_share)
            qkv = g(x, L["self_qkv"], self._sms - kv_share)
            v = qkv[:, 2 * (qkv.shape[1] // 3):]
            x = self._row(v, L["self_o"])
        elif self.collective == "fused":
            # the sum is inside self o's launch: fork before it, so the cross k/v launch runs
            # beside it and fills the SMs while it waits for the other ranks
            qkv = g(x, L["self_qkv"])
            v = qkv[:, 2 * (qkv.shape[1] // 3):]
            side.wait_stream(cur)
            x = self._row(v, L["self_o"])
            with torch.cuda.stream(side):
                kv = g(ctx, L["cross_kv"], max(self._sms // 2, 1))
        else:
            qkv = g(x, L["self_qkv"])
            v = qkv[:, 2 * (qkv.shape[1] // 3):]
            partial = g(self._row_input(v, L["self_o"]), L["self_o"])
            side.wait_stream(cur)  # after self o's GEMM, alongside its collective
            with torch.cuda.stream(side):
                kv = g(ctx, L["cross_kv"], max(self._sms // 2, 1))
            x = self._reduce(partial)
        g(x, L["cross_q"])
        cur.wait_stream(side)
        cv = kv[:, kv.shape[1] // 2:]
        x = self._row(cv, L["cross_o"])
        h = g(x, L["ffn_up"])
        x = self._row(h, L["ffn_down"])
        return x

    def block_forward(self, blk: int, x: torch.Tensor, ctx: torch.Tensor) -> torch.Tensor:
        """x, ctx: ``[M, dim]`` replicated on every rank; returns the new replicated x."""
        if self.concurrent and not self.fuse_qkv and x.is_cuda:
            return self._block_forward_concurrent(blk, x, ctx)
        if self.concurrent and self.fuse_qkv and x.is_cuda:
            return self._block_forward_fused_overlapped(blk, x, ctx)
        L = {l.name: l for l in self.layers[blk]}
        g = self._g
        # self attention: q, k, v column-parallel; the v shard stands in for the attention output
        if self.fuse_qkv:
            qkv = g(x, L["self_qkv"])
            v = qkv[:, 2 * (qkv.shape[1] // 3):]
        else:
            g(x, L["self_q"])
            g(x, L["self_k"])
            v = g(x, L["self_v"])
        x = self._row(v, L["self_o"])
        # cross attention: q on x, k and v on the context
        g(x, L["cross_q"])
        if self.fuse_qkv:
            kv = g(ctx, L["cross_kv"])
            cv = kv[:, kv.shape[1] // 2:]
        else:
            g(ctx, L["cross_k"])
            cv = g(ctx, L["cross_v"])
        x = self._row(cv, L["cross_o"])
        # FFN
        h = g(x, L["ffn_up"])
        x = self._row(h, L["ffn_down"])
        return x

    def _row_input(self, col_out: torch.Tensor, row_layer: ShardedLinear) -> torch.Tensor:
        """Activation slice a row-parallel linear consumes.

        With even column shards the column-parallel output of this rank IS that
        slice.  When the row cut (whole groups) does not coincide with the column
        cut, the slice is gathered first.
        """
        k0, k1 = row_layer.k_range
        if self.world == 1:
            return col_out
        c0, c1 = self._local_cols(row_layer.full_shape[0])
        if (c0, c1) == (k0, k1):
            return col_out
        import torch.distributed as dist

        parts = [torch.empty_like(col_out) for _ in range(self.world)]
        dist.all_gather(parts, col_out.contiguous(), group=self.process_group)
        return torch.cat(parts, dim=-1)[:, k0:k1].contiguous()

    def forward(self, x: torch.Tensor, ctx: Optional[torch.Tensor] = None) -> torch.Tensor:
        ctx = x if ctx is None else ctx
        for blk in range(self.blocks):
            x = self.block_forward(blk, x, ctx)
        return x
