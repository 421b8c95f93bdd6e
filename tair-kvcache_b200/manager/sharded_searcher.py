"""Hash-range-sharded matching across GPUs: one process per GPU, one index shard per process.

The index of one instance is split by key-hash range over the ranks of a torch.distributed group; every
rank hashes and submits its own batch of requests.  One exchange step per query:

  prefix match    all-gather of keys  ->  every shard counts leading keys, skipping keys it does not own
                  ->  all-reduce(MIN) of the per-request lengths;
  sliding window  all-gather of keys  ->  every shard writes the servable flag of the keys it owns
                  ->  all-reduce(MAX) of the flag bytes  ->  local window search over the flags.

Both equal MetaSearcher::PrefixMatch / ReverseRollSlideWindowMatch
(kv_cache_manager/manager/meta_searcher.cc:120-145, 196-265) on the unsharded index because every key has
exactly one owner.  The collectives run over the group's backend (NCCL on GPUs); data lands in local
buffers before any kernel reads it.

A third way, "route", sends every key only to the shard that owns it (an all-to-all of 8-byte keys bucketed on
the device) and gets one flag byte per key back (a second all-to-all), after which both matchers run locally
over the flag bytes: the traffic per key is 9 bytes whatever the number of shards.
"""
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .. import _cabi

_MASK64 = (1 << 64) - 1


def shard_of_keys(keys: np.ndarray, shard_count: int) -> np.ndarray:
    """Owner shard of each int64 key: floor(fmix64(key) * shard_count / 2**64).  Host twin of the device rule."""
    out = np.empty(len(keys), dtype=np.int32)
    for i, k in enumerate(np.asarray(keys, dtype=np.int64).tolist()):
        k &= _MASK64
        k ^= k >> 33
        k = (k * 0xFF51AFD7ED558CCD) & _MASK64
        k ^= k >> 33
        k = (k * 0xC4CEB9FE1A85EC53) & _MASK64
        k ^= k >> 33
        out[i] = (k * shard_count) >> 64
    return out


class CudaShardBackend:
    """The shard-local work, on the GPU through the C ABI."""

    def __init__(self, max_keys: int, device: torch.device, avail_mask: int = _cabi.AVAIL_ALL):
        from .block_index import BlockIndex
        self.index = BlockIndex(max_keys, device)
        self.device = self.index.device
        self.avail_mask = avail_mask

    def upsert_owned(self, keys, value_word, shard_count, shard_rank):
        _cabi.call("kvcm_b200_index_upsert_sharded", self.index.handle, keys.data_ptr(), None, value_word,
                   keys.numel(), shard_count, shard_rank, None, self.index._s())

    def prefix_owned(self, keys, key_off, mask_off, shard_count, shard_rank):
        n_req = key_off.numel() - 1
        out = torch.empty(n_req, dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_match_prefix_sharded", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req,
                   mask_off.data_ptr() if mask_off is not None else None, None, self.avail_mask, shard_count,
                   shard_rank, out.data_ptr(), self.index._s())
        return out

    def write_snapshot(self, keys, storage_class, shard_count, shard_rank):
        """The flags a write looks at for the keys this shard owns, 0 for the others."""
        out = torch.zeros(max(keys.numel(), 1), dtype=torch.uint8, device=self.device)
        _cabi.call("kvcm_b200_write_snapshot_sharded", self.index.handle, keys.data_ptr(), keys.numel(), self.avail_mask,
                   int(storage_class), shard_count, shard_rank, out.data_ptr(), self.index._s())
        return out[:keys.numel()]

    def start_write_owned(self, keys, key_off, flags, skip, storage_class, shard_count, shard_rank, table_full=None):
        """StartWriteCache of the whole (gathered) batch on this shard: the answers for every request, the new
        locations of the keys this shard owns.  Returns (offset, mask, n_new, added, new_off)."""
        n_req = key_off.numel() - 1
        dev = self.device
        need = int(_cabi.lib().kvcm_b200_start_write_workspace_bytes(keys.numel(), n_req))
        if need < 0:
            raise ValueError("too many keys for one StartWriteCache batch")
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        offset = torch.empty(max(n_req, 1), dtype=torch.int32, device=dev)
        n_new = torch.empty(max(n_req, 1), dtype=torch.int32, device=dev)
        mask = torch.empty(max(keys.numel(), 1), dtype=torch.uint8, device=dev)
        added = torch.zeros(max(keys.numel(), 1), dtype=torch.uint8, device=dev)
        new_off = torch.zeros(n_req + 1, dtype=torch.int64, device=dev)
        flags = flags if flags.numel() > 0 else torch.zeros(1, dtype=torch.uint8, device=dev)
        _cabi.call("kvcm_b200_start_write_sharded", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req,
                   keys.numel(), self.avail_mask, int(storage_class), flags.data_ptr(),
                   skip.data_ptr() if skip is not None else None, shard_count, shard_rank, ws.data_ptr(), need,
                   offset.data_ptr(), mask.data_ptr(), n_new.data_ptr(), added.data_ptr(), new_off.data_ptr(),
                   table_full.data_ptr() if table_full is not None else None, self.index._s())
        ws.record_stream(torch.cuda.current_stream(dev))
        return offset[:n_req], mask, n_new[:n_req], added, new_off

    def finish_write_owned(self, keys, key_off, added, new_off, success_off, storage_class, shard_count, shard_rank):
        n_req = key_off.numel() - 1
        out = torch.zeros(max(n_req, 1), dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_finish_write_sharded", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req,
                   added.data_ptr(), new_off.data_ptr(), success_off.data_ptr(), None, int(storage_class), shard_count,
                   shard_rank, out.data_ptr(), self.index._s())
        return out[:n_req]

    def servable_flags(self, keys, shard_count=1, shard_rank=0):
        out = torch.empty(keys.numel(), dtype=torch.uint8, device=self.device)
        _cabi.call("kvcm_b200_batch_get_sharded", self.index.handle, keys.data_ptr(), keys.numel(), self.avail_mask,
                   shard_count, shard_rank, out.data_ptr(), self.index._s())
        return out

    def sw_from_flags(self, flags, key_off, sw):
        n_req = key_off.numel() - 1
        out = torch.empty(n_req, dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_match_sw_from_flags", flags.data_ptr(), key_off.data_ptr(), n_req, sw, out.data_ptr(),
                   self.index._s())
        return out

    def prefix_from_flags(self, flags, key_off, mask_off):
        n_req = key_off.numel() - 1
        out = torch.empty(n_req, dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_match_prefix_from_flags", flags.data_ptr(), key_off.data_ptr(), n_req,
                   mask_off.data_ptr() if mask_off is not None else None, None, out.data_ptr(), self.index._s())
        return out

    def route_count(self, keys, shard_count):
        counts = torch.empty(shard_count, dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_route_count", keys.data_ptr(), keys.numel(), shard_count, counts.data_ptr(),
                   self.index._s())
        return counts

    def route_scatter(self, keys, shard_count, cursor):
        bucketed = torch.empty_like(keys)
        pos = torch.empty(keys.numel(), dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_route_scatter", keys.data_ptr(), keys.numel(), shard_count, cursor.data_ptr(),
                   bucketed.data_ptr(), pos.data_ptr(), self.index._s())
        return bucketed, pos

    def gather_bytes(self, src, pos):
        out = torch.empty(pos.numel(), dtype=torch.uint8, device=self.device)
        _cabi.call("kvcm_b200_gather_bytes", src.data_ptr(), pos.data_ptr(), pos.numel(), out.data_ptr(),
                   self.index._s())
        return out

    # ---- routed exchange over peer memory ----
    def route_area_create(self, capacity_keys):
        import ctypes
        area = ctypes.c_void_p()
        _cabi.bind_device(self.device.index)
        _cabi.call("kvcm_b200_route_area_create", int(capacity_keys), ctypes.byref(area))
        return area

    def route_area_destroy(self, area):
        _cabi.call("kvcm_b200_route_area_destroy", area)

    def route_dispatch(self, area, keys, matrix):
        cursor = torch.empty(matrix.shape[0], dtype=torch.int32, device=self.device)
        pos = torch.empty(keys.numel(), dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_route_dispatch", area, keys.data_ptr(), keys.numel(), matrix.ctypes.data,
                   cursor.data_ptr(), pos.data_ptr(), self.index._s())
        return pos

    def route_answer(self, area, matrix):
        _cabi.call("kvcm_b200_route_answer", self.index.handle, area, matrix.ctypes.data, self.avail_mask,
                   self.index._s())

    def route_collect(self, area, pos):
        out = torch.empty(pos.numel(), dtype=torch.uint8, device=self.device)
        _cabi.call("kvcm_b200_route_collect", area, pos.data_ptr(), pos.numel(), out.data_ptr(), self.index._s())
        return out

    def sw_direct(self, keys, key_off, sw):
        n_req = key_off.numel() - 1
        out = torch.empty(n_req, dtype=torch.int32, device=self.device)
        _cabi.call("kvcm_b200_match_sw", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req, sw,
                   self.avail_mask, out.data_ptr(), self.index._s())
        return out


class GatheredRequests:
    """All ranks' requests after the exchange step, reusable for several queries on the same keys."""

    def __init__(self, keys, csr, per_req, first, n_req):
        self.keys, self.csr, self.per_req, self.first, self.n_req = keys, csr, per_req, first, n_req


class ShardedWriteSessions:
    """This rank's answers of a sharded StartWriteCache (offset / mask / n_new / added as in WriteSessions) and the
    gathered batch its FinishWriteCache works on."""

    def __init__(self, offset, mask, n_new, added, all_keys, csr, all_added, new_off, first, n_req, max_req,
                 storage_class):
        self.offset, self.mask, self.n_new, self.added = offset, mask, n_new, added
        self.all_keys, self.csr, self.all_added, self.new_off = all_keys, csr, all_added, new_off
        self.first, self.n_req, self.max_req, self.storage_class = first, n_req, max_req, storage_class

    @property
    def session_lengths(self) -> torch.Tensor:
        """Session keys per request of this rank."""
        lens = self.new_off[1:] - self.new_off[:-1]
        return lens[self.first:self.first + self.n_req]


class RoutedFlags:
    """The servable flag of each of this rank's keys, fetched from the owning shards; reusable for several
    queries on the same keys."""

    def __init__(self, flags, key_off, mask_off):
        self.flags, self.key_off, self.mask_off = flags, key_off, mask_off


class ShardedMetaSearcher:
    """Collective front end: every rank of `group` calls each method with its own requests.

    mode "exchange": one all-gather of keys and one min / max all-reduce per query (works on any backend).
    mode "peer":     after `attach_peers()` every rank probes the owner shard of each key directly over NVLink
                     (CUDA IPC mappings, plain peer loads): queries need no collective at all; only writes do.
    mode "route":    every key goes to its owner and one flag byte comes back (two all-to-alls per batch of
                     requests, shared by the prefix and the window query when `Route()` is called once).
    mode "route_peer": the same exchange without a transport: after `attach_route_areas()` the dispatch kernel
                     stores the keys into the owners' inboxes and the owners store the flag bytes back, both
                     over NVLink peer memory; the ranks meet at two one-word all-reduces per batch.
                     `route_capacity` = keys one inbox / answer buffer holds (at least the largest batch of a
                     rank, plus the imbalance of the split); `route_areas` = batches that may be in flight at
                     once (one per stream the caller routes on)."""

    def __init__(self, backend, group: Optional[dist.ProcessGroup] = None, mode: str = "exchange",
                 route_capacity: int = 0, route_areas: int = 1):
        self.backend = backend
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = backend.device
        self.mode = mode
        self.areas = []
        if mode == "peer":
            self.attach_peers()
        if mode == "route_peer":
            self.attach_route_areas(route_capacity, route_areas)

    def attach_route_areas(self, capacity_keys: int, count: int = 1) -> None:
        """Allocate `count` exchange areas, exchange their IPC handles and map the peers' (one-time set-up)."""
        import ctypes
        if capacity_keys <= 0:
            raise _cabi.KvcmError(_cabi.KVCM_EC_BADARGS, "attach_route_areas: route_capacity")
        asked = [None] * self.world  # one capacity for all ranks: the largest any of them asks for
        dist.all_gather_object(asked, int(capacity_keys), group=self.group)
        capacity_keys = max(asked)
        self._tick = torch.zeros(1, dtype=torch.int32, device=self.device)
        for _ in range(count):
            area = self.backend.route_area_create(capacity_keys)
            exp = _cabi.RouteExport()
            _cabi.call("kvcm_b200_route_area_export", area, ctypes.byref(exp))
            blobs = [None] * self.world
            dist.all_gather_object(blobs, bytes(exp), group=self.group)
            arr = (_cabi.RouteExport * self.world)()
            for r, blob in enumerate(blobs):
                ctypes.memmove(ctypes.addressof(arr[r]), blob, ctypes.sizeof(_cabi.RouteExport))
            _cabi.bind_device(self.device.index)
            _cabi.call("kvcm_b200_route_area_attach", area, self.world, self.rank, arr)
            self.areas.append(area)
        self.mode = "route_peer"

    def detach_route_areas(self) -> None:
        """Unmap the peers' areas and free this rank's; every rank calls it, with no batch in flight."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for area in self.areas:
            _cabi.call("kvcm_b200_route_area_detach", area)
        dist.barrier(group=self.group)
        for area in self.areas:
            self.backend.route_area_destroy(area)
        self.areas = []
        self.mode = "exchange"

    def attach_peers(self) -> None:
        """Exchange the shards' IPC handles and map every shard into this process (one-time set-up)."""
        import ctypes
        exp = _cabi.IndexExport()
        _cabi.call("kvcm_b200_index_export", self.backend.index.handle, ctypes.byref(exp))
        blobs = [None] * self.world
        dist.all_gather_object(blobs, bytes(exp), group=self.group)
        arr = (_cabi.IndexExport * self.world)()
        for r, blob in enumerate(blobs):
            ctypes.memmove(ctypes.addressof(arr[r]), blob, ctypes.sizeof(_cabi.IndexExport))
        _cabi.bind_device(self.device.index)
        _cabi.call("kvcm_b200_index_attach_peers", self.backend.index.handle, self.world, self.rank, arr)
        self.mode = "peer"

    def detach_peers(self) -> None:
        """Unmap the peers' shards; every rank calls it (after a barrier) before any shard is freed."""
        dist.barrier(group=self.group)
        _cabi.call("kvcm_b200_index_detach_peers", self.backend.index.handle)
        dist.barrier(group=self.group)
        self.mode = "exchange"

    def _publish_writes(self) -> None:
        """Writes of all shards become visible to every rank's next query."""
        if self.mode == "peer":
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)

    # ---- exchange -----------------------------------------------------------------------------
    def _gather_requests(self, keys: torch.Tensor, key_off: torch.Tensor, per_req: Optional[torch.Tensor]
                         ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], int, int]:
        """All ranks' requests as one CSR batch with fixed per-rank strides.

        Rank r contributes max_req + 1 requests over a segment of max_keys keys: its real requests, then empty
        ones up to max_req, then one filler request that covers the zero padding of its segment (so the CSR
        stays contiguous).  Returns (all keys, all offsets, all per-request values, max_req, my first request)."""
        n_req, n_keys = key_off.numel() - 1, int(keys.numel())
        sizes = torch.tensor([n_req, n_keys], dtype=torch.int64, device=self.device)
        all_sizes = torch.empty(self.world * 2, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(all_sizes, sizes, group=self.group)
        all_sizes = all_sizes.view(self.world, 2).cpu()
        max_req, max_keys = int(all_sizes[:, 0].max()), int(all_sizes[:, 1].max())
        seg_keys = torch.zeros(max(max_keys, 1), dtype=torch.int64, device=self.device)
        seg_keys[:n_keys] = keys
        seg_off = torch.full((max_req + 1,), n_keys, dtype=torch.int64, device=self.device)
        seg_off[:n_req + 1] = key_off
        all_keys = torch.empty(self.world * seg_keys.numel(), dtype=torch.int64, device=self.device)
        all_off = torch.empty(self.world * (max_req + 1), dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(all_keys, seg_keys, group=self.group)
        dist.all_gather_into_tensor(all_off, seg_off, group=self.group)
        stride = seg_keys.numel()
        base = torch.arange(self.world, dtype=torch.int64, device=self.device).repeat_interleave(max_req + 1) * stride
        csr = torch.cat([all_off + base, torch.tensor([self.world * stride], dtype=torch.int64, device=self.device)])
        all_per_req = None
        if per_req is not None:
            seg = torch.zeros(max_req + 1, dtype=per_req.dtype, device=self.device)
            seg[:n_req] = per_req
            all_per_req = torch.empty(self.world * (max_req + 1), dtype=per_req.dtype, device=self.device)
            dist.all_gather_into_tensor(all_per_req, seg, group=self.group)
        return all_keys, csr, all_per_req, max_req, self.rank * (max_req + 1)

    def _gather_keys(self, keys: torch.Tensor) -> torch.Tensor:
        n = torch.tensor([keys.numel()], dtype=torch.int64, device=self.device)
        counts = torch.empty(self.world, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(counts, n, group=self.group)
        counts = counts.cpu().tolist()
        seg = torch.zeros(max(max(counts), 1), dtype=torch.int64, device=self.device)
        seg[:keys.numel()] = keys
        out = torch.empty(self.world * seg.numel(), dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(out, seg, group=self.group)
        return torch.cat([out[r * seg.numel(): r * seg.numel() + c] for r, c in enumerate(counts)])

    # ---- route --------------------------------------------------------------------------------
    def Route(self, keys: torch.Tensor, key_off: torch.Tensor, mask_off: Optional[torch.Tensor] = None,
              area: int = 0) -> RoutedFlags:
        """Dispatch this rank's keys to their owners, look them up there, combine the answers back in key order.
        `area` (mode "route_peer") picks the exchange area: batches in flight at once use different ones, and
        every rank routes its batches in the same order.

        Stream rule: the whole call runs on torch's CURRENT stream.  The kernels are launched on it, and the
        collectives between them are enqueued by torch.distributed, which orders NCCL's work after and before the
        current stream only; that ordering is all that keeps "dispatch | answer | collect" apart (a peer's keys
        have landed before this rank answers, its answers have landed before this rank collects).  A caller that
        wants two batches in flight wraps each call in `with torch.cuda.stream(s):` and gives each its own area;
        launching the kernels on any other stream than the current one would let an answer run ahead of the
        keys it answers."""
        keys, key_off = keys.contiguous(), key_off.contiguous()
        counts = self.backend.route_count(keys, self.world)
        matrix = torch.empty(self.world * self.world, dtype=torch.int32, device=self.device)
        dist.all_gather_into_tensor(matrix, counts, group=self.group)
        matrix = matrix.view(self.world, self.world).cpu()
        if self.mode == "route_peer":
            h_counts = np.ascontiguousarray(matrix.numpy().astype(np.uint32))
            pos = self.backend.route_dispatch(self.areas[area], keys, h_counts)
            dist.all_reduce(self._tick, group=self.group)  # every rank's keys have landed
            self.backend.route_answer(self.areas[area], h_counts)
            dist.all_reduce(self._tick, group=self.group)  # every owner's answers have landed
            return RoutedFlags(self.backend.route_collect(self.areas[area], pos), key_off, mask_off)
        send = matrix[self.rank].tolist()      # my keys per owner
        recv = matrix[:, self.rank].tolist()   # keys I own, per asking rank
        cursor = (torch.cumsum(counts, 0, dtype=torch.int32) - counts).contiguous()
        bucketed, pos = self.backend.route_scatter(keys, self.world, cursor)
        asked = torch.empty(sum(recv), dtype=torch.int64, device=self.device)
        dist.all_to_all_single(asked, bucketed, recv, send, group=self.group)
        answers = self.backend.servable_flags(asked, 1, 0)
        back = torch.empty(keys.numel(), dtype=torch.uint8, device=self.device)
        dist.all_to_all_single(back, answers, send, recv, group=self.group)
        return RoutedFlags(self.backend.gather_bytes(back, pos), key_off, mask_off)

    # ---- operators ----------------------------------------------------------------------------
    def upsert(self, keys: torch.Tensor, value_word: int) -> None:
        """Every rank contributes keys; each key is stored on the shard that owns it."""
        self.backend.upsert_owned(self._gather_keys(keys.contiguous()), value_word, self.world, self.rank)
        self._publish_writes()

    # ---- write side ---------------------------------------------------------------------------
    def StartWriteCache(self, keys: torch.Tensor, key_off: torch.Tensor, storage_class: int,
                        table_full: Optional[torch.Tensor] = None) -> "ShardedWriteSessions":
        """CacheManager::StartWriteCache (kv_cache_manager/manager/cache_manager.cc:334-430) for every rank's
        requests at once, answered as if the reference had served them one after the other in the order (rank,
        request): one all-gather of the requests, one all-reduce (bytewise maximum) of the flags each key's owner
        sees, then every rank computes the same block masks and write sessions and merges the new locations of the
        keys it owns.  Returns this rank's answers and what FinishWriteCache of the batch needs."""
        n_req = key_off.numel() - 1
        all_keys, csr, _, max_req, first = self._gather_requests(keys.contiguous(), key_off.contiguous(), None)
        skip = torch.zeros(self.world * (max_req + 1), dtype=torch.uint8, device=self.device)
        skip[max_req::max_req + 1] = 1  # every rank's last entry covers the padding of its segment
        flags = self.backend.write_snapshot(all_keys, storage_class, self.world, self.rank)
        dist.all_reduce(flags, op=dist.ReduceOp.MAX, group=self.group)
        offset, mask, n_new, added, new_off = self.backend.start_write_owned(
            all_keys, csr, flags, skip, storage_class, self.world, self.rank, table_full)
        self._publish_writes()
        k0 = int(csr[first].item())
        return ShardedWriteSessions(offset[first:first + n_req], mask[k0:k0 + keys.numel()], n_new[first:first + n_req],
                                    added[k0:k0 + keys.numel()], all_keys, csr, added, new_off, first, n_req, max_req,
                                    int(storage_class))

    def FinishWriteCache(self, sessions: "ShardedWriteSessions", success_off: torch.Tensor) -> torch.Tensor:
        """CacheManager::FinishWriteCache (:432-501) for the sessions of one StartWriteCache batch: success_off is
        this rank's BlockMaskOffset per request over its session keys.  Every rank makes the transitions of the
        session keys it owns; returns this rank's result code per request."""
        seg = torch.zeros(sessions.max_req + 1, dtype=torch.int64, device=self.device)
        seg[:sessions.n_req] = success_off
        all_success = torch.empty(self.world * (sessions.max_req + 1), dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(all_success, seg, group=self.group)
        codes = self.backend.finish_write_owned(sessions.all_keys, sessions.csr, sessions.all_added, sessions.new_off,
                                                all_success, sessions.storage_class, self.world, self.rank)
        dist.all_reduce(codes, op=dist.ReduceOp.MAX, group=self.group)
        self._publish_writes()
        return codes[sessions.first:sessions.first + sessions.n_req]

    def Gather(self, keys: torch.Tensor, key_off: torch.Tensor, mask_off: Optional[torch.Tensor] = None
               ) -> GatheredRequests:
        """The exchange step on its own: all-gather of every rank's keys (and mask offsets).  Pass the result to
        PrefixMatch / ReverseRollSlideWindowMatch to run several queries on one exchange."""
        all_keys, csr, all_mask, _, first = self._gather_requests(keys.contiguous(), key_off.contiguous(), mask_off)
        return GatheredRequests(all_keys, csr, all_mask, first, key_off.numel() - 1)

    def PrefixMatch(self, keys, key_off: Optional[torch.Tensor] = None, mask_off: Optional[torch.Tensor] = None
                    ) -> torch.Tensor:
        if self.mode == "peer":  # the attached handle resolves every key at its owner: a purely local call
            return self.backend.prefix_owned(keys.contiguous(), key_off.contiguous(), mask_off, 1, 0)
        if self.mode in ("route", "route_peer") or isinstance(keys, RoutedFlags):
            r = keys if isinstance(keys, RoutedFlags) else self.Route(keys, key_off, mask_off)
            return self.backend.prefix_from_flags(r.flags, r.key_off, r.mask_off)
        g = keys if isinstance(keys, GatheredRequests) else self.Gather(keys, key_off, mask_off)
        lens = self.backend.prefix_owned(g.keys, g.csr, g.per_req, self.world, self.rank)
        dist.all_reduce(lens, op=dist.ReduceOp.MIN, group=self.group)
        return lens[g.first:g.first + g.n_req]

    def ReverseRollSlideWindowMatch(self, keys, key_off: Optional[torch.Tensor] = None, sw_size: int = 0
                                    ) -> torch.Tensor:
        if sw_size <= 0:
            raise _cabi.KvcmError(_cabi.KVCM_EC_BADARGS, "ReverseRollSlideWindowMatch")
        if self.mode == "peer":
            return self.backend.sw_direct(keys.contiguous(), key_off.contiguous(), sw_size)
        if self.mode in ("route", "route_peer") or isinstance(keys, RoutedFlags):
            r = keys if isinstance(keys, RoutedFlags) else self.Route(keys, key_off, None)
            return self.backend.sw_from_flags(r.flags, r.key_off, sw_size)
        g = keys if isinstance(keys, GatheredRequests) else self.Gather(keys, key_off, None)
        flags = self.backend.servable_flags(g.keys, self.world, self.rank)
        dist.all_reduce(flags, op=dist.ReduceOp.MAX, group=self.group)
        base = self.backend.sw_from_flags(flags, g.csr, sw_size)
        return base[g.first:g.first + g.n_req]
