"""Multi-GPU use of the path, one process per GPU (torch.distributed, NCCL over NVLink on GPUs, gloo in the
CPU tests).  The reference is single-GPU (kvarn-port has no collective call site), so this layer is new:

* one long sequence: the context is cut into contiguous tile ranges, one per rank, each rank holding its range
  as a local cache of its own; every rank attends its range, exports the log-sum-exp partial (m, l, o_rot)
  per query head, one all-gather moves the partials (q_heads * (head_dim + 2) floats per rank) and every rank
  merges them.  The open tile lives on the last rank, which also receives the appends.
* many independent sequences: whole sequences are dealt to ranks, longest first onto the least loaded rank;
  no communication on the data path.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

TILE = 128


def tile_ranges(kv_len: int, world: int) -> List[Tuple[int, int]]:
    """Token range [begin, end) of every rank: whole tiles, contiguous, as even as possible; the remainder
    (open tile) goes to the last rank.  Ranks beyond the number of tiles get empty ranges."""
    tiles = kv_len // TILE
    per, extra = divmod(tiles, world)
    out, t = [], 0
    for r in range(world):
        n = per + (1 if r < extra else 0)
        out.append((t * TILE, (t + n) * TILE))
        t += n
    b, _ = out[-1]
    out[-1] = (b, kv_len)
    return out


def deal_sequences(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time greedy: indices of the sequences each rank serves."""
    load = [0] * world
    owner: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(lengths)), key=lambda j: -lengths[j]):
        r = min(range(world), key=lambda k: (load[k], k))
        owner[r].append(i)
        load[r] += lengths[i]
    return owner


def pack_partial(m, l, o):
    """(m [QH], l [QH], o [QH, D]) -> one [QH, D + 2] tensor for a single all-gather."""
    import torch

    return torch.cat([m.unsqueeze(1), l.unsqueeze(1), o], dim=1).contiguous()


def unpack_partials(buf):
    """[R, QH, D + 2] -> m [R, QH], l [R, QH], o [R, QH, D] (contiguous copies)."""
    return buf[..., 0].contiguous(), buf[..., 1].contiguous(), buf[..., 2:].contiguous()


def all_gather_partials(packed, group=None):
    """One collective per layer call: every rank ends with [world, QH, D + 2]."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    out = torch.empty((world * packed.shape[0],) + tuple(packed.shape[1:]), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(out, packed, group=group)  # rank r's block lands at rows [r * QH, (r + 1) * QH)
    return out.view((world,) + tuple(packed.shape))


class ShardedDecode:
    """Decode attention of one sequence whose cache is range-sharded over the ranks of `group`.
    `layer` is this rank's local KvarnLayer (its tile range, local positions 0..).  Three launches per call:
    attention with partial export into the send buffer, one all-gather, the merge kernel."""

    def __init__(self, layer, group=None):
        import torch
        import torch.distributed as dist

        self.layer, self.group = layer, group
        self.world = dist.get_world_size(group)
        n = layer.q_heads * (layer.head_dim + 2)
        self.send = torch.empty(n, dtype=torch.float32, device=layer.device)
        self.recv = torch.empty(self.world * n, dtype=torch.float32, device=layer.device)

    def attn_decode(self, q, local_pos, scale: float, local_len_max: int, out):
        import torch.distributed as dist

        from . import cache

        self.layer.attn_decode_partial_packed(q, local_pos, scale, local_len_max, self.send)
        dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        return cache.merge_partials_packed(self.recv, self.world, self.layer.q_heads, self.layer.head_dim, out)


class ShardedChunk:
    """A verify step or a prefill chunk over a sequence whose cache is range-sharded over the ranks of `group`: the new
    rows are appended on the rank that owns the open tile (the last one), every rank attends its own range
    (kvb_attn_chunk_partial), one all-gather moves the partials (tokens * q_heads * (head_dim + 2) floats per rank),
    every rank merges.  `max_tokens` sizes the buffers."""

    def __init__(self, layer, max_tokens: int, group=None):
        import torch
        import torch.distributed as dist

        self.layer, self.group = layer, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.per_token = layer.q_heads * (layer.head_dim + 2)
        self.send = torch.empty(max_tokens * self.per_token, dtype=torch.float32, device=layer.device)
        self.recv = torch.empty(self.world * max_tokens * self.per_token, dtype=torch.float32, device=layer.device)

    def attend(self, q, k, v, local_positions, scale: float, local_len_max: int, out):
        """q: [tokens, q_heads, D] (the same on every rank); k, v: the new rows (used on the owner rank only);
        local_positions: int32 [tokens] on the device -- on the owner the positions of the new rows in its cache, on
        the other ranks the position of their last token, repeated.
        When the rows divide by the ranks, the partials are not gathered everywhere: every rank receives the partials
        of its share of the rows (one all-to-all), merges them, and the finished rows are gathered -- (N-1)/N of a
        partial plus (N-1)/N of an output per rank instead of N-1 partials."""
        import torch
        import torch.distributed as dist

        from . import cache

        tokens = int(q.shape[0])
        n = tokens * self.per_token
        if self.rank == self.world - 1:
            self.layer.append(k, v, local_positions)
        self.layer.attn_chunk_partial_packed(q, local_positions, scale, local_len_max, self.send[:n])
        rows, D = tokens * self.layer.q_heads, self.layer.head_dim
        if self.world > 1 and rows % self.world == 0 and rows >= 8 * self.world:
            share = rows // self.world
            m, l, o = self.send[:rows], self.send[rows:2 * rows], self.send[2 * rows:n]
            rm, rl, ro = self.recv[:rows], self.recv[rows:2 * rows], self.recv[2 * rows:n]  # [world][share] and [world][share][D]
            dist.all_to_all_single(rm, m, group=self.group)
            dist.all_to_all_single(rl, l, group=self.group)
            dist.all_to_all_single(ro, o, group=self.group)
            mine = cache.merge_partials(rm.view(self.world, share), rl.view(self.world, share), ro.view(self.world, share, D), out.dtype)
            dist.all_gather_into_tensor(out.view(rows, D), mine, group=self.group)
            return out
        dist.all_gather_into_tensor(self.recv[:self.world * n], self.send[:n], group=self.group)
        return cache.merge_partials_packed(self.recv[:self.world * n], self.world, tokens * self.layer.q_heads, self.layer.head_dim,
                                           out.view(tokens * self.layer.q_heads, self.layer.head_dim))


class PeerRing:
    """Ring buffers for kvb_attn_decode_sharded: one buffer per rank that every rank can write (peer memory).
    `PeerRing.symmetric(...)` allocates it with torch's symmetric memory over the process group (NVLink peer
    mappings); `PeerRing.loopback(...)` builds a single-process stand-in whose "peers" are local buffers (tests)."""

    def __init__(self, local_buf, peer_ptrs, rank: int, world: int, device, max_spins: int = 0, keep=(), rows: int = 0):
        import ctypes as C

        import torch

        from . import capi

        self.local_buf, self.rank, self.world, self._keep = local_buf, rank, world, keep
        self.peer_ptrs = (C.c_void_p * world)(*[int(p) for p in peer_ptrs])
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        self.c = capi.kvb_peer_ring(peer_bufs=self.peer_ptrs, local_buf=local_buf.data_ptr(),
                                    state=self.state.data_ptr(), rank=rank, world=world, max_spins=max_spins, rows=rows)
        self._C = C

    @staticmethod
    def nbytes(world: int, q_heads: int, head_dim: int) -> int:
        from . import capi

        return capi.load().kvb_peer_ring_bytes(world, q_heads, head_dim)

    @classmethod
    def symmetric(cls, q_heads: int, head_dim: int, device, group=None, max_spins: int = 0, tokens: int = 1):
        """`tokens`: query tokens per call the ring must hold (1 = decode only, 8 = verify steps too)."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        buf = symm_mem.empty(cls.nbytes(world, tokens * q_heads, head_dim) // 4, dtype=torch.float32, device=device)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize()
        dist.barrier(group)  # every rank's buffer is zeroed before anybody may push
        return cls(buf, [int(p) for p in hdl.buffer_ptrs], rank, world, device, max_spins, keep=(hdl,), rows=tokens * q_heads)

    @classmethod
    def loopback(cls, q_heads: int, head_dim: int, device, world: int = 1, rank: int = 0, max_spins: int = 0, tokens: int = 1):
        import torch

        bufs = [torch.zeros(cls.nbytes(world, tokens * q_heads, head_dim) // 4, dtype=torch.float32, device=device) for _ in range(world)]
        return cls(bufs[rank], [b.data_ptr() for b in bufs], rank, world, device, max_spins, keep=tuple(bufs), rows=tokens * q_heads)


class RingShardedDecode:
    """Range-sharded decode with the partial exchange done by the kernels themselves (peer stores + arrival flags)."""

    def __init__(self, layer, ring: PeerRing):
        self.layer, self.ring = layer, ring

    def attn_decode(self, q, local_pos, scale: float, local_len_max: int, out):
        import ctypes as C

        import torch

        from . import capi

        L = self.layer
        capi.check(capi.load().kvb_attn_decode_sharded(C.byref(L.c), C.c_void_p(q.data_ptr()), C.c_void_p(local_pos.data_ptr()), scale,
                                                       local_len_max, C.c_void_p(L.workspace(local_len_max, 1).data_ptr()),
                                                       C.byref(self.ring.c), C.c_void_p(out.data_ptr()),
                                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    def attn_verify(self, q, k, v, local_positions, scale: float, local_len_max: int, out, owner: bool):
        """A verify step of 1..8 rows: the owner of the open tile appends the rows (k, v), every rank attends its own
        range and the reduce kernel exchanges the partials over the ring (kvb_attn_rows_sharded): three launches on
        the owner, two elsewhere, no collective.  local_positions as for ShardedChunk.attend."""
        import ctypes as C

        import torch

        from . import capi

        L = self.layer
        rows = int(q.shape[0])
        if owner:
            L.append(k, v, local_positions)
        capi.check(capi.load().kvb_attn_rows_sharded(C.byref(L.c), C.c_void_p(q.data_ptr()), C.c_void_p(local_positions.data_ptr()), rows,
                                                     scale, local_len_max, C.c_void_p(L.workspace(local_len_max, rows).data_ptr()),
                                                     C.byref(self.ring.c), C.c_void_p(out.data_ptr()),
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out
