"""Partitioning of the compressed-attention work across the GPUs of one box.

The unit of work is a lane: one (sequence, KV head) pair.  A lane's packed codes, norms and
fp16 sink/recent tokens are read by exactly one CTA group, and the attention outputs of the
query heads that share that KV head depend on nothing else, so lanes can be dealt to ranks
with no data-path collective.  Two plans:

* by sequence (``plan_lanes(..., split_heads=False)``): whole sequences per rank; nothing is
  exchanged.  This is what ``bench.py --gpus N`` times.
* by sequence and KV head (``split_heads=True``): used when there are fewer sequences than
  ranks; each rank then holds the caches of its KV heads only and the per-head outputs are
  gathered once per step (``gather_heads``), the only collective on the path.

  ``FusedGather`` is the same exchange without a collective: the decode kernel's merge step stores each
  rank's heads straight into every rank's landing buffer (peer-mapped device memory, plain 64-bit stores that carry
  their own arrival mark), and the next kernel on the consumer's stream collects them.

``job_time_ms`` is the barrier-free max over ranks that multi-GPU timings must use.
"""

from __future__ import annotations

from dataclasses import dataclass

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


@dataclass(frozen=True)
class LanePlan:
    """Half-open ranges of sequences and KV heads owned by one rank."""
    seq_begin: int
    seq_end: int
    head_begin: int
    head_end: int

    @property
    def n_lanes(self) -> int:
        return (self.seq_end - self.seq_begin) * (self.head_end - self.head_begin)


def _even_range(n: int, parts: int, index: int) -> tuple[int, int]:
    """Range `index` of `n` items dealt to `parts` owners, sizes differing by at most one."""
    base, extra = divmod(n, parts)
    begin = index * base + min(index, extra)
    return begin, begin + base + (1 if index < extra else 0)


def plan_lanes(n_sequences: int, n_kv_heads: int, world: int, rank: int, split_heads: bool | None = None) -> LanePlan:
    """Lanes of rank `rank` out of `world`.

    With ``split_heads`` None the plan splits by sequence whenever every rank can get at least one
    sequence, otherwise by (sequence, head group): ranks are arranged as `n_sequences` rows of
    ``world // n_sequences`` head groups, which must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_sequences < 1 or n_kv_heads < 1:
        raise ValueError("need at least one sequence and one KV head")
    if split_heads is None:
        split_heads = n_sequences < world
    if not split_heads:
        b, e = _even_range(n_sequences, world, rank)
        return LanePlan(b, e, 0, n_kv_heads)
    if world % n_sequences:
        raise ValueError(f"{world} ranks cannot be arranged as {n_sequences} sequences x head groups")
    groups = world // n_sequences
    if n_kv_heads % groups:
        raise ValueError(f"{n_kv_heads} KV heads do not split into {groups} equal groups")
    seq, grp = divmod(rank, groups)
    per = n_kv_heads // groups
    return LanePlan(seq, seq + 1, grp * per, (grp + 1) * per)


def gather_heads(local_out: torch.Tensor, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """Concatenate per-rank attention outputs (B, H_q_local, 1, D) along the head axis.

    Only needed under a head-split plan; ranks of one sequence row must form `group` in head order."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)


class _DeviceView:
    """A span of raw device memory that ``torch.as_tensor`` can wrap (CUDA array interface, version 2)."""

    def __init__(self, address: int, shape: tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (address, False), "version": 2,
                                         "strides": None}


_TYPESTR = {torch.float16: ("<f2", 2), torch.float32: ("<f4", 4), torch.bfloat16: (None, 2)}


class SlotLedger:
    """Reuse rule of the gather slots, as host-side bookkeeping: with more than one rank a peer may already be writing
    call n + 1 into a slot while this rank still reads call n from it, unless the two calls use different slots.  So
    more than one rank needs at least two slots, and the same slot may not take two decode calls in a row."""

    def __init__(self, world: int, n_buffers: int):
        if n_buffers < 1:
            raise ValueError("n_buffers must be at least 1")
        if world > 1 and n_buffers < 2:
            raise ValueError("with more than one rank a gather needs at least two slots (n_buffers >= 2): a peer may "
                             "overwrite a slot this rank is still reading")
        self.world, self.n_buffers, self._last = world, n_buffers, None

    def use(self, i: int) -> None:
        if not 0 <= i < self.n_buffers:
            raise IndexError(f"slot {i} of {self.n_buffers}")
        if self.world > 1 and i == self._last:
            raise RuntimeError(f"slot {i} was also the previous decode call's slot: a peer could overwrite the result "
                               "while it is being read; alternate between slots")
        self._last = i


class FusedGather:
    """Every rank's landing buffers, mapped into every rank (ranks = GPUs of one node).

    ``n_buffers`` independent slots (one per layer in flight is the usual choice).  A slot is a landing buffer of 64-bit
    words {4 bytes of the result, 32-bit epoch} that every rank's merge steps write into, this rank's epoch array (how many
    calls it has made into the slot) and a plain result ``(batch, heads_total, d)`` of ``dtype``.  A decode call given
    ``slot(i)`` sends its heads into slot ``i`` of every rank; the gather is complete on this rank once every word of its
    landing buffer carries this rank's own epoch (every rank makes the same calls with the same sizes).  The consumer
    waits for that, and unpacks the words into ``result(i)``, inside the next decode call -
    ``attend(..., after=arrived(i))``, no launch in between - or with ``wait(i)``, a small kernel on the current stream,
    before a reader that is not one of this package's kernels.  Epochs are kept on the device, so every launch takes the
    same arguments every step and a step can be captured in a CUDA graph.

    A slot may take its next call only when every rank has collected the previous one, which holds when slots are used
    in turn (no slot twice in a row) and every call waits for its predecessor's gather.
    """

    def __init__(self, batch: int, heads_total: int, d: int, dtype: torch.dtype, n_buffers: int, head_offset: int,
                 n_local_heads: int, n_local_kv_heads: int, device: torch.device, group: dist.ProcessGroup | None = None):
        if dtype not in _TYPESTR:
            raise TypeError(f"unsupported result dtype {dtype}")
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _lib.TQ_MAX_PEERS:
            raise ValueError(f"at most {_lib.TQ_MAX_PEERS} ranks")
        self._ledger = SlotLedger(self.world, n_buffers)
        self.shape, self.dtype, self.n_buffers, self.device = (batch, heads_total, d), dtype, n_buffers, device
        lib = _lib.lib()
        elem = _TYPESTR[dtype][1]
        self._words = batch * heads_total * d * elem // 4
        groups = int(lib.tq_gather_groups(batch, n_local_heads, n_local_kv_heads))
        if groups < 1:
            raise ValueError(f"{n_local_heads} query heads over {n_local_kv_heads} KV heads")
        pad = lambda n: (n + 255) // 256 * 256
        self._ll_bytes = pad(self._words * 8)
        self._out_off = n_buffers * self._ll_bytes                                   # plain results (local use only)
        self._out_bytes = pad(self._words * 4)
        self._epoch_off = self._out_off + n_buffers * self._out_bytes                # epoch arrays (local use only)
        self._epoch_bytes = pad(groups * 4)
        total = self._epoch_off + n_buffers * self._epoch_bytes
        with torch.cuda.device(device):
            base = C.c_void_p()
            handle = C.create_string_buffer(64)
            _lib.check(lib.tq_peer_buffer_create(total, C.byref(base), handle))
            self._own = base.value
            mine = (device.index if device.index is not None else torch.cuda.current_device(), bytes(handle.raw),
                    (batch, n_local_heads, n_local_kv_heads))
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            self._bases, self._opened = [], []
            failure = None
            if any(e[2] != mine[2] for e in everyone):     # the completion rule counts on every rank making the same calls
                failure = f"rank {self.rank}: ranks hold different numbers of heads: {[e[2] for e in everyone]}"
            for r, (peer_dev, h, _) in enumerate(everyone):
                if failure:
                    break
                if r == self.rank:
                    self._bases.append(self._own)
                    continue
                p = C.c_void_p()
                rc = lib.tq_peer_buffer_open(h, peer_dev, C.byref(p))
                if rc != 0:
                    failure = f"rank {self.rank}: cannot map rank {r}'s buffer: " + lib.tq_last_error().decode("utf-8", "replace")
                    break
                self._bases.append(p.value)
                self._opened.append(p.value)
            # every rank learns of any rank's failure before anybody waits for anybody
            reports = [None] * self.world
            dist.all_gather_object(reports, failure, group=group)
            if any(reports):
                self.close()
                raise RuntimeError("; ".join(m for m in reports if m))
        self._structs = []
        for i in range(n_buffers):
            g = _lib.PeerGather()
            g.n_peers, g.heads_total, g.head_offset = self.world, heads_total, head_offset
            g.dtype, g.shape = dtype, (batch, d)                    # (Python attributes: attend checks its call against them)
            for r, b in enumerate(self._bases):
                g.ll[r] = b + i * self._ll_bytes
            g.epochs = self._own + self._epoch_off + i * self._epoch_bytes
            self._structs.append(g)
        self._results = [self._view(i) for i in range(n_buffers)]
        if dist.get_world_size(group) > 1:
            dist.barrier(group=group)          # nobody writes before everybody has mapped everybody

    def _view(self, i: int) -> torch.Tensor:
        b, h, d = self.shape
        addr = self._own + self._out_off + i * self._out_bytes
        typestr = _TYPESTR[self.dtype][0]
        if typestr is None:                    # bfloat16 has no array-interface code: wrap as int16, reinterpret
            t = torch.as_tensor(_DeviceView(addr, (b, h, d), "<i2"), device=self.device).view(torch.bfloat16)
        else:
            t = torch.as_tensor(_DeviceView(addr, (b, h, d), typestr), device=self.device)
        return t

    def slot(self, i: int) -> "_lib.PeerGather":
        """The argument for ``TurboQuantKVCache.attend(..., gather=...)``; call it once per decode call (it records the
        slot's use and refuses the same slot twice in a row when there are peers)."""
        self._ledger.use(i)
        return self._structs[i]

    def arrived(self, i: int) -> tuple[int, int, int, int]:
        """The ``after=`` argument of a later ``attend`` on this stream: that kernel waits for slot ``i`` to be complete
        here and fills ``result(i)``."""
        return (self._own + i * self._ll_bytes, self._own + self._epoch_off + i * self._epoch_bytes, self._words,
                self._own + self._out_off + i * self._out_bytes)

    def wait(self, i: int) -> None:
        """Order the current stream behind the arrival of every rank's heads of the latest decode call on slot ``i``;
        fills ``result(i)``."""
        _lib.check(_lib.launch(self.device, "tq_gather_wait", *self.arrived(i), _lib.stream_ptr(self.device)))

    def result(self, i: int) -> torch.Tensor:
        """(batch, heads_total, d) view of this rank's copy of slot ``i`` (complete once the slot has been waited for)."""
        return self._results[i]

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (call on every rank, after a barrier and a device sync)."""
        lib = _lib.lib()
        with torch.cuda.device(self.device):
            for p in self._opened:
                lib.tq_peer_buffer_close(p)
            self._opened = []
            if self._own:
                lib.tq_peer_buffer_destroy(self._own)
                self._own = 0


def job_time_ms(local_ms: float, device: torch.device | None = None, group: dist.ProcessGroup | None = None) -> float:
    """Max over ranks of a device-measured duration."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(local_ms)
    t = torch.tensor([local_ms], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
