"""Sharding of one decode layer over the GPUs of a node, one process per GPU.

(row, kv head) items are independent, so the layer splits with no data-path exchange until the
outputs are put together:

  heads: rank r owns kv heads [r*Hkv/N, (r+1)*Hkv/N) and the query heads of those groups; its pool
         is [page][Hkv/N][token][d]; allocator, block table, lengths and plan are replicated.
  batch: rank r owns a contiguous range of batch rows with all heads (used when Hkv < N, and for
         data-parallel replicas of a larger global batch).

The exchange step is an all-gather of the fp16 outputs.  `gather_outputs` does it with the
process group (NCCL on GPUs, gloo in the CPU tests) and returns the full [B][Hq][d] layout.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_begin: int
    kv_end: int
    q_begin: int
    q_end: int

    @property
    def num_kv_heads(self):
        return self.kv_end - self.kv_begin

    @property
    def num_q_heads(self):
        return self.q_end - self.q_begin


def shard_heads(rank, world, num_q_heads, num_kv_heads):
    """KV-head sharding.  The group size is unchanged, so the same kernel instance runs on every rank."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    if num_q_heads % num_kv_heads:
        raise ValueError("num_q_heads must be a multiple of num_kv_heads")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} kv heads do not divide over {world} ranks; shard the batch instead")
    kv, group = num_kv_heads // world, num_q_heads // num_kv_heads
    return HeadShard(rank, world, rank * kv, (rank + 1) * kv, rank * kv * group, (rank + 1) * kv * group)


def shard_batch(rank, world, batch):
    """Contiguous row range [begin, end) of rank `rank`; the first batch % world ranks get one more row."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def local_query(q_full, shard):
    """q [B][Hq][d] -> this rank's [B][Hq/N][d] (contiguous)."""
    return q_full[:, shard.q_begin:shard.q_end].contiguous()


def local_kv(k_or_v, shard):
    """K or V tokens [n][Hkv][d] -> this rank's [n][Hkv/N][d] (contiguous), the append input of its cache."""
    return k_or_v[:, shard.kv_begin:shard.kv_end].contiguous()


def gather_outputs(out_local, mode, group=None, rows=None):
    """All-gather of per-rank outputs into the full layout.

    mode "heads": out_local is [B][Hq/N][d] on every rank -> [B][Hq][d].
    mode "batch": out_local is [B_r][Hq][d] -> [sum B_r][Hq][d]; `rows` lists every rank's B_r when
    they differ (ragged shards are padded to the largest for the collective).
    """
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return out_local
    if mode == "heads":
        b, hq_local, d = out_local.shape
        gathered = torch.empty((world * b, hq_local, d), dtype=out_local.dtype, device=out_local.device)
        dist.all_gather_into_tensor(gathered, out_local.contiguous(), group=group)   # rank-major concatenation
        return gathered.view(world, b, hq_local, d).permute(1, 0, 2, 3).reshape(b, world * hq_local, d)
    if mode == "batch":
        rows = list(rows) if rows is not None else [out_local.shape[0]] * world
        widest = max(rows)
        padded = out_local
        if out_local.shape[0] < widest:
            padded = torch.zeros((widest,) + tuple(out_local.shape[1:]), dtype=out_local.dtype, device=out_local.device)
            padded[:out_local.shape[0]] = out_local
        gathered = torch.empty((world * widest,) + tuple(padded.shape[1:]), dtype=out_local.dtype, device=out_local.device)
        dist.all_gather_into_tensor(gathered, padded.contiguous(), group=group)
        gathered = gathered.view((world, widest) + tuple(padded.shape[1:]))
        return torch.cat([gathered[r, :rows[r]] for r in range(world)], dim=0)
    raise ValueError("mode must be 'heads' or 'batch'")


class GatherGroup:
    """Gathered outputs without a collective call: every rank's decode kernel stores its rows into
    every peer's buffer (peer stores over NVLink), a one-warp kernel behind it raises this rank's flag on
    every peer, and `wait` / `wait_epoch` enqueue the bounded wait for all ranks' flags.  One process per
    GPU; the IPC handles travel through the torch process group."""

    def __init__(self, out_bytes, group=None):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import _lib
        self._lib, self._C = _lib, C
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out_bytes = out_bytes
        # Set-up is collective: every step below is followed by an exchange of "did it work", so that a
        # rank that cannot allocate or map a peer makes ALL ranks raise instead of leaving the others
        # waiting in a collective.
        self._h = None
        err = None
        n = _lib.lib().pd_gather_handle_bytes()
        mine = C.create_string_buffer(n)
        try:
            h = C.c_void_p()
            _lib.check(_lib.lib().pd_gather_create(self.world, self.rank, out_bytes, C.byref(h)))
            self._h = h
            _lib.check(_lib.lib().pd_gather_export(h, mine))
        except Exception as e:
            err = e
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, (mine.raw, err is None), group=group)
            if err is None and all(ok for _, ok in handles):
                try:
                    _lib.check(_lib.lib().pd_gather_connect(self._h, b"".join(hb for hb, _ in handles)))
                except Exception as e:
                    err = e
            elif err is None:
                err = RuntimeError("a peer could not create its gather block")
            oks = [None] * self.world
            dist.all_gather_object(oks, err is None, group=group)   # also: everyone has mapped every block
            if err is None and not all(oks):
                err = RuntimeError("a peer could not map the gather blocks")
        if err is not None:
            self.close()
            raise err
        torch.cuda.synchronize()

    def close(self):
        if getattr(self, "_h", None):
            self._lib.lib().pd_gather_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:          # interpreter shutdown: the module is already gone
            pass

    def decode(self, dtype, params, row_stride_heads, head_offset=0, row_offset=0, stream=0, num_pages=0, sync=False):
        """One layer with its rows stored into every rank's buffer.  sync=False: returns after the announcement
        is queued; `wait` / `wait_epoch` wait for the peers whenever the caller wants.  sync=True: the kernel
        behind the decode also waits for all ranks' rows (one launch fewer)."""
        fn = self._lib.lib().pd_paged_decode_gather_sync if sync else self._lib.lib().pd_paged_decode_gather
        self._lib.check(fn(int(dtype), self._C.byref(params), num_pages, self._h, row_stride_heads, head_offset,
                           row_offset, stream))

    def wait(self, stream=0):
        self._lib.check(self._lib.lib().pd_gather_wait(self._h, stream))

    def wait_epoch(self, epoch, stream=0):
        """Wait (bounded) for the rows of step `epoch`; see `epoch` for the current step number."""
        self._lib.check(self._lib.lib().pd_gather_wait_epoch(self._h, epoch, stream))

    @property
    def epoch(self):
        return self._lib.lib().pd_gather_epoch(self._h)

    def buffer_ptr(self, which=-1):
        """Device pointer of the local gathered buffer (which = step mod 4, -1 = the one the last decode filled)."""
        return self._lib.lib().pd_gather_buffer(self._h, which)
