"""Batched iov copy and the debug CRC against the oracle's restatement of the reference's per-iov loops."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _segments_from_iovs(iovs, string_ptr, direction):
    """iovs: list of (device tensor or None, size, ignore).  Returns a device tensor of kvcm_b200_seg_t."""
    n = len(iovs)
    arr = (_cabi.Iov * n)()
    for i, (t, size, ign) in enumerate(iovs):
        arr[i].type = 1
        arr[i].ignore = 1 if ign else 0
        arr[i].base = t.data_ptr() if t is not None else None
        arr[i].size = size
    segs = (_cabi.Seg * n)()
    n_segs, span = ctypes.c_int32(), ctypes.c_uint64()
    _cabi.call("kvcm_b200_iovs_to_segments", ctypes.addressof(arr), n, string_ptr, direction, ctypes.addressof(segs),
               ctypes.addressof(n_segs), ctypes.addressof(span))
    raw = np.frombuffer(bytes(segs), dtype=np.uint8)[:n_segs.value * ctypes.sizeof(_cabi.Seg)].copy()
    return torch.from_numpy(raw).to(DEV), n_segs.value, span.value


def test_block_of_layer_iovs_put_and_get_match_the_reference_loop():
    """One block = layer_num x (K, V) iovs (kv_cache_manager/client/include/common.h:99-116), some ignored,
    odd sizes and unaligned bases included."""
    rng = np.random.default_rng(3)
    _cabi.bind_device(0)
    sizes = [4096, 4096, 100, 7, 65536 + 16, 0, 33000, 4096, 1 << 20, 12345]
    ignore = [False, False, False, True, False, False, True, False, False, False]
    host = [rng.integers(0, 256, size=s + 3, dtype=np.uint8) for s in sizes]
    dev = [torch.from_numpy(h).to(DEV) for h in host]
    # odd-indexed iovs start 3 bytes into their allocation: unaligned bases
    views = [d[3:3 + s] if i % 2 else d[:s] for i, (d, s) in enumerate(zip(dev, sizes))]
    hviews = [h[3:3 + s] if i % 2 else h[:s] for i, (h, s) in enumerate(zip(host, sizes))]
    total = sum(sizes)
    string = torch.zeros(total, dtype=torch.uint8, device=DEV)
    iovs = [(v if s > 0 else None, s, ign) for v, s, ign in zip(views, sizes, ignore)]
    segs, n_segs, span = _segments_from_iovs(iovs, string.data_ptr(), 0)
    assert span == total and n_segs == sum(1 for s, g in zip(sizes, ignore) if s > 0 and not g)
    _cabi.call("kvcm_b200_copy_segments", segs.data_ptr(), n_segs, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    # the same list with its size stated takes the bulk-copy ring (mean segment 129 KiB): identical bytes
    ring_string = torch.zeros_like(string)
    ring_segs, _, _ = _segments_from_iovs(iovs, ring_string.data_ptr(), 0)
    _cabi.call("kvcm_b200_copy_segments_sized", ring_segs.data_ptr(), n_segs, total,
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(ring_string, string)
    want = np.zeros(total, dtype=np.uint8)
    oracle.copy_iovs([(hv if s > 0 else None, s, g) for hv, s, g in zip(hviews, sizes, ignore)], want, 0)
    assert np.array_equal(string.cpu().numpy(), want)

    # Get: block string -> fresh iovs
    fresh = [torch.zeros_like(d) for d in dev]
    fviews = [f[3:3 + s] if i % 2 else f[:s] for i, (f, s) in enumerate(zip(fresh, sizes))]
    segs, n_segs, _ = _segments_from_iovs([(v if s > 0 else None, s, g) for v, s, g in zip(fviews, sizes, ignore)],
                                          string.data_ptr(), 1)
    _cabi.call("kvcm_b200_copy_segments", segs.data_ptr(), n_segs, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for i, (fv, hv, g) in enumerate(zip(fviews, hviews, ignore)):
        got = fv.cpu().numpy()
        assert np.array_equal(got, np.zeros_like(got) if g else hv), i
    for f, s, i in zip(fresh, sizes, range(len(sizes))):  # nothing outside the iov was touched
        outside = torch.cat([f[:3], f[3 + s:]]) if i % 2 else f[s:]
        assert not outside.any()


def test_many_small_segments_and_empty_list():
    _cabi.bind_device(0)
    n, size = 5000, 256
    src = torch.randint(0, 256, (n * size,), dtype=torch.uint8, device=DEV)
    dst = torch.zeros_like(src)
    perm = torch.randperm(n).tolist()
    segs = (_cabi.Seg * n)()
    for i, j in enumerate(perm):
        segs[i].dst = dst.data_ptr() + j * size
        segs[i].src = src.data_ptr() + i * size
        segs[i].bytes = size
    d = torch.from_numpy(np.frombuffer(bytes(segs), dtype=np.uint8).copy()).to(DEV)
    _cabi.call("kvcm_b200_copy_segments", d.data_ptr(), n, None)
    _cabi.call("kvcm_b200_copy_segments", d.data_ptr(), 0, None)
    torch.cuda.synchronize()
    assert torch.equal(dst.view(n, size)[perm], src.view(n, size))


def test_iov_crc_known_answers(match_kat):
    _cabi.bind_device(0)
    cases = match_kat["crc"][0]["cases"]
    bufs = [torch.tensor(list(c["text"].encode()), dtype=torch.uint8, device=DEV) for c in cases]
    for buf, c in zip(bufs, cases):
        seg = (_cabi.Seg * 1)()
        seg[0].src = buf.data_ptr()
        seg[0].bytes = buf.numel()
        d = torch.from_numpy(np.frombuffer(bytes(seg), dtype=np.uint8).copy()).to(DEV)
        out = torch.zeros(1, dtype=torch.int32, device=DEV)
        # SdkBufferCheckUtil::GetIovsCrc: cal_byte_size = min(min_cal_byte_size, size / 2)
        cal = min(c["min_cal_bytes"], buf.numel() // 2)
        _cabi.call("kvcm_b200_iov_crc", d.data_ptr(), 1, cal, out.data_ptr(), None)
        torch.cuda.synchronize()
        assert (out.item() & 0xFFFFFFFF) == int(c["crc"], 16)


def test_iov_crc_random_against_oracle():
    _cabi.bind_device(0)
    rng = np.random.default_rng(9)
    host = [rng.integers(0, 256, size=int(rng.integers(8, 5000)), dtype=np.uint8) for _ in range(300)]
    dev = [torch.from_numpy(h).to(DEV) for h in host]
    segs = (_cabi.Seg * len(dev))()
    for i, t in enumerate(dev):
        segs[i].src = t.data_ptr()
        segs[i].bytes = t.numel()
    d = torch.from_numpy(np.frombuffer(bytes(segs), dtype=np.uint8).copy()).to(DEV)
    out = torch.zeros(len(dev), dtype=torch.int32, device=DEV)
    _cabi.call("kvcm_b200_iov_crc", d.data_ptr(), len(dev), 4, out.data_ptr(), None)
    torch.cuda.synchronize()
    got = out.cpu().numpy().view(np.uint32)
    want = np.array([oracle.iov_crc(h, 4) for h in host], dtype=np.uint32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("n_segs,seg_bytes", [(3, 5 << 20), (700, 96 * 1024 + 48), (40, 8192), (1, 1 << 20)])
def test_bulk_ring_path_of_sized_copies(n_segs, seg_bytes):
    """Few large segments (chunks of one segment shared by several CTAs), more segments than CTAs, sizes that are
    not multiples of the 32 KiB chunk or of 16 bytes, and one segment whose ends are not 16-byte aligned."""
    _cabi.bind_device(0)
    gen = torch.Generator(device=DEV).manual_seed(n_segs)
    pad = 64
    src = torch.randint(0, 256, (n_segs * (seg_bytes + pad),), dtype=torch.uint8, device=DEV, generator=gen)
    dst = torch.zeros_like(src)
    sizes = [seg_bytes - (7 if i % 3 == 1 else 0) for i in range(n_segs)]
    shift = [5 if i == n_segs - 1 and n_segs > 1 else 0 for i in range(n_segs)]  # one unaligned segment
    segs = (_cabi.Seg * n_segs)()
    for i in range(n_segs):
        segs[i].dst = dst.data_ptr() + i * (seg_bytes + pad) + shift[i]
        segs[i].src = src.data_ptr() + i * (seg_bytes + pad) + shift[i]
        segs[i].bytes = sizes[i]
    d = torch.from_numpy(np.frombuffer(bytes(segs), dtype=np.uint8).copy()).to(DEV)
    _cabi.call("kvcm_b200_copy_segments_sized", d.data_ptr(), n_segs, sum(sizes), None)
    torch.cuda.synchronize()
    a, b = dst.view(n_segs, -1).cpu().numpy(), src.view(n_segs, -1).cpu().numpy()
    for i in range(n_segs):
        assert np.array_equal(a[i, shift[i]:shift[i] + sizes[i]], b[i, shift[i]:shift[i] + sizes[i]]), i
        assert not a[i, :shift[i]].any() and not a[i, shift[i] + sizes[i]:].any(), i  # nothing outside a segment
    count = (ctypes.c_uint32 * 1)()
    _cabi.call("kvcm_b200_copy_wait_timeouts", ctypes.addressof(count))
    assert count[0] == 0
