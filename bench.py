"""Benchmark of the KVCM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2|c3|c1]

Default workload (`c2`): Llama-3-8B-shaped paged-KV transfer on one GPU - 32 layers x (K,V) pools of
65,536 pages of 16 tokens x 1024 bf16, 2,048 transfer blocks of 4 pages each addressed through a random
non-contiguous page table, gathered into contiguous device staging and scattered back.  One step = one
gather plus one scatter of all blocks.  `value` is GB/s of algorithmic bytes (2 x payload per direction:
every payload byte is read once and written once), inputs resident in HBM.  `e2e` is the same metric
through the Python operator API with the staging buffers in pinned host memory, i.e. with the
device<->host traffic of a real save / load inside the timed region.

With N > 1 (torchrun) every rank moves its own tensor-parallel slice of the same shape: no data-path
collective, weak scaling, time = max over ranks.

`--impl reference` times the CPU restatement of the same step (oracle/, all host threads) on a bounded
sample of the workload, on rank 0 only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

# The default of 8 hardware work queues per process lets two of this program's many CUDA streams (two per
# end-to-end leg, two copy streams of the library, two of the two-stream match step) land on one queue, where their
# kernels then run one after the other.  32 is the driver's maximum; it must be set before CUDA is initialised.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "kv_block_gather_scatter_bandwidth"
UNIT = "GB/s"
# DRAM bytes read + written per algorithmic byte of MoveRowsBulkKernel, from the ncu capture summarised in
# profiles/move_rows_bulk_llama8b_reduced_ncu_full.md (4.2505 GB per 4.2950 GB launch); traffic grows in
# proportion to the blocks moved, so the full-size figure is this ratio times the launch's algorithmic bytes.
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = (2.147519 + 2.102969) / 4.294967296
# the same ratio for the bulk segment copy (profiles/copy_segments_bulk_256_blocks_ncu_full.md)
IOV_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = (2.148165 + 2.106079) / 4.294967296

WORKLOADS = {
    # name: layers, kv pools per layer, page tokens, bytes per token per pool, pages per pool, blocks, pages per block
    "c2": dict(desc="llama3-8b paged-KV gather+scatter, 32 layers x (K,V), 8 kv heads x 128 bf16, page 16, "
                    "2048 blocks x 64 tokens, random page table, device staging",
               n_pools=64, page_tokens=16, token_bytes=2048, pool_pages=65536, n_blocks=2048, pages_per_block=4),
    "c3": dict(desc="llama3-70b TP=8 slice per rank, 80 layers x (K,V), 1 kv head x 128 bf16, page 32, "
                    "8192 blocks x 128 tokens per rank, random page table, device staging",
               n_pools=160, page_tokens=32, token_bytes=256, pool_pages=65536, n_blocks=8192, pages_per_block=4),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"



class Ctx:
    """This process's place in the job: one process per GPU, one process group for the whole run."""

    def __init__(self):
        import torch
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        self.device = torch.device("cuda", self.local)
        torch.cuda.set_device(self.device)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()

    def max_over_ranks(self, values):
        """Element-wise maximum of a list of floats over the ranks (device-timed figures: the slowest rank counts)."""
        import torch
        if self.world == 1:
            return list(values)
        import torch.distributed as dist
        t = torch.tensor(list(values), dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampling of this GPU's SM clock and throttle reasons (read-only).  The sampler is started well
    before the timed region (nvidia-smi needs a moment to come up) and only the samples whose timestamps fall
    inside [mark_begin(), mark_end()] are kept."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid = uuid if str(uuid).startswith("GPU-") else "GPU-" + str(uuid)
        self.proc = None
        self.path = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "10"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            time.sleep(0.5)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside, everything, reasons, sm_max = [], [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    mhz = float(parts[1])
                    sm_max = float(parts[2])
                except ValueError:
                    continue
                everything.append(mhz)
                if self.t0 is None or self.t0 - 0.01 <= ts <= (self.t1 or ts) + 0.01:
                    inside.append(mhz)
                    for name, val in zip(names, parts[4:8]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
        os.unlink(self.path)
        use = inside or everything
        if use:
            out.update(sm_mhz=statistics.median(use), sm_max_mhz=sm_max, reasons=sorted(reasons),
                       samples=len(inside), samples_around=len(everything))
        return out


# ----------------------------------------------------------------------------------------------
# workload
# ----------------------------------------------------------------------------------------------
def build_transfer_workload(cfg, device, seed):
    """Pools, page table, staging slot order on `device`.  Pool size shrinks if the GPU cannot hold it
    (the referenced pages and the bytes moved stay the same)."""
    import torch
    n_pools, page_bytes = cfg["n_pools"], cfg["page_tokens"] * cfg["token_bytes"]
    n_blocks, ppb = cfg["n_blocks"], cfg["pages_per_block"]
    payload = n_blocks * n_pools * ppb * page_bytes
    free, _ = torch.cuda.mem_get_info(device)
    pool_pages = cfg["pool_pages"]
    while pool_pages > 2 * n_blocks * ppb and n_pools * pool_pages * page_bytes + payload + (6 << 30) > free:
        pool_pages //= 2
    gen = torch.Generator(device=device).manual_seed(seed)
    pools = []
    for _ in range(n_pools):
        # random 32-bit patterns = random bf16 bit patterns, NaN and Inf payloads included
        t = torch.empty(pool_pages * page_bytes // 4, dtype=torch.int32, device=device)
        t.random_(-(1 << 31), (1 << 31) - 1, generator=gen)
        pools.append(t)
    ptrs = torch.tensor([p.data_ptr() for p in pools], dtype=torch.int64, device=device)
    rng = np.random.default_rng(seed)
    table = torch.from_numpy(rng.permutation(pool_pages)[:n_blocks * ppb].astype(np.int32)).to(device)
    slots = torch.from_numpy(rng.permutation(n_blocks).astype(np.int32)).to(device)
    staging = torch.zeros(payload // 4, dtype=torch.int32, device=device)
    return dict(pools=pools, ptrs=ptrs, table=table, slots=slots, staging=staging, pool_pages=pool_pages,
                page_bytes=page_bytes, payload=payload, n_pools=n_pools, n_blocks=n_blocks, ppb=ppb)


def verify_gather(w):
    """Every staged tile equals a torch gather of the pools (all blocks, all pools): the check shares no code
    with the kernel under test."""
    import torch
    st = w["staging"].view(w["n_blocks"], w["n_pools"], w["ppb"], -1)
    table = w["table"].long().view(w["n_blocks"], w["ppb"])
    slots = w["slots"].long()
    for p in range(w["n_pools"]):
        if not torch.equal(st[slots, p], w["pools"][p].view(w["pool_pages"], -1)[table]):
            return False
    return True


def verify_scatter(w, scatter):
    """The scatter direction at full size, in a form that can fail: every staged word is changed, the blocks are
    scattered, then every referenced page must equal its staged tile and a sample of unreferenced pages must be
    untouched.  (Scattering back what was just gathered would rewrite the pools with their own content.)"""
    import torch
    rng = np.random.default_rng(3)
    referenced = np.zeros(w["pool_pages"], dtype=bool)
    referenced[w["table"].cpu().numpy()] = True
    others = np.flatnonzero(~referenced)
    others = torch.from_numpy(rng.choice(others, size=min(256, len(others)), replace=False)).to(w["staging"].device) \
        if len(others) else None
    before = [pool.view(w["pool_pages"], -1)[others].clone() for pool in w["pools"]] if others is not None else []
    w["staging"].bitwise_xor_(0x5A5A5A5A)
    scatter()
    torch.cuda.synchronize()
    ok = verify_gather(w)  # pools[table] == staging[slots] again, now with the new content
    for pool, b in zip(w["pools"], before):
        ok = ok and torch.equal(pool.view(w["pool_pages"], -1)[others], b)
    return bool(ok)


def transfer_config(cfg, payload):
    """The `config` object of the transfer workloads: what is moved, nothing about how a run went, so that the GPU
    arm and the CPU arm print the same object."""
    return {"workload": cfg["desc"], "pool_pages": cfg["pool_pages"], "payload_bytes_per_direction": payload,
            "l2": "inputs (%.1f GiB staged per direction) far exceed the 126 MB L2; no flush needed"
                  % (payload / 2 ** 30)}


def full_payload(cfg):
    return cfg["n_blocks"] * cfg["n_pools"] * cfg["pages_per_block"] * cfg["page_tokens"] * cfg["token_bytes"]


def run_cpu_transfer(cfg, threads, steps, warmup, budget_s=20.0, max_payload=None):
    """The CPU restatement of one gather + scatter step on a bounded sample (host memory): as many of the
    workload's blocks as fit a quarter of the free host memory (pools twice the payload, staging once) and
    `max_payload`, up to the whole workload."""
    import psutil

    from oracle import kvcm_oracle as oracle
    n_pools, page_bytes, ppb = cfg["n_pools"], cfg["page_tokens"] * cfg["token_bytes"], cfg["pages_per_block"]
    block_bytes = n_pools * ppb * page_bytes
    room = psutil.virtual_memory().available // 4 // 3
    if max_payload is not None:
        room = min(room, max_payload)
    n_blocks = int(max(1, min(cfg["n_blocks"], room // block_bytes)))
    pool_pages = 2 * n_blocks * ppb
    rng = np.random.default_rng(0xB2000002)
    # uniform-random bytes: one random 16 MiB piece per pool laid end to end (memcpy speed does not depend on
    # the values, and drawing tens of GiB from a generator would take longer than the measurement)
    pools = []
    for _ in range(n_pools):
        piece = rng.integers(0, 256, size=min(16 << 20, pool_pages * page_bytes), dtype=np.uint8)
        pools.append(np.resize(piece, pool_pages * page_bytes))
    table = rng.permutation(pool_pages)[:n_blocks * ppb].astype(np.int32)
    slots = rng.permutation(n_blocks).astype(np.int32)
    staging = np.zeros(n_blocks * block_bytes, dtype=np.uint8)
    payload = staging.nbytes

    def step():
        oracle.move_rows(pools, staging, table, slots, ppb, page_bytes, 0, threads=threads)
        oracle.move_rows(pools, staging, table, slots, ppb, page_bytes, 1, threads=threads)

    for _ in range(warmup):
        step()
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    total = sum(times)
    gbs = 4.0 * payload * len(times) / total / 1e9
    sample = "%d of %d blocks (%.2f GiB payload per direction), %d pools of %d pages in host memory, %d steps" % (
        n_blocks, cfg["n_blocks"], payload / 2 ** 30, n_pools, pool_pages, len(times))
    return gbs, 1e3 * total / len(times), sample, len(times)


# ----------------------------------------------------------------------------------------------
# prefix-match side workload (second half of the metric), small and quick
# ----------------------------------------------------------------------------------------------
def build_prefix_workload(seed=0xB2000001, n_req=4096, n_prior_blocks=200000, bs=64):
    """CPU-runnable prefix-match configuration: uint32 tokens uniform in [0,151936), lengths uniform 512-8192,
    half of the requests reuse a random-length prefix of an earlier sequence, index pre-filled with the
    hashes of n_prior_blocks prior blocks."""
    rng = np.random.default_rng(seed)
    prior, n = [], 0
    while n < n_prior_blocks:
        t = rng.integers(0, 151936, size=int(rng.integers(512, 8193)), dtype=np.int64).astype(np.uint32)
        prior.append(t)
        n += len(t) // bs
    seqs = list(prior)
    reqs = []
    for _ in range(n_req):
        t = rng.integers(0, 151936, size=int(rng.integers(512, 8193)), dtype=np.int64).astype(np.uint32)
        if rng.random() < 0.5:
            src = seqs[int(rng.integers(0, len(seqs)))]
            m = int(rng.integers(1, min(len(t), len(src)) + 1))
            t[:m] = src[:m]
        reqs.append(t)
        seqs.append(t)

    def csr(seq_list):
        off = np.zeros(len(seq_list) + 1, dtype=np.int64)
        np.cumsum([len(s) for s in seq_list], out=off[1:])
        return np.concatenate(seq_list), off

    return csr(prior), csr(reqs), n_prior_blocks, bs


def run_prefix_gpu(device, steps, warmup):
    import torch
    from tair_kvcache_b200.manager import (BatchMetaSearcher, BlockIndex, GenKeyVectorBatch, encode_locations,
                                           key_offsets)
    (ptoks, poff), (toks, off), n_prior, bs = build_prefix_workload()
    pko = key_offsets(poff, bs)
    pkeys = GenKeyVectorBatch(torch.from_numpy(ptoks.view(np.int32)).to(device), torch.from_numpy(poff).to(device), bs,
                              torch.from_numpy(pko).to(device), int(pko[-1]))[:n_prior]
    index = BlockIndex(n_prior, device)
    index.upsert(pkeys, None, encode_locations([(3, 4)]))
    searcher = BatchMetaSearcher(index)
    ko = key_offsets(off, bs)
    n_keys = int(ko[-1])
    h_toks = torch.from_numpy(toks.view(np.int32)).pin_memory()
    h_off = torch.from_numpy(off).pin_memory()
    h_ko = torch.from_numpy(ko).pin_memory()
    d_toks, d_off, d_ko = h_toks.to(device), h_off.to(device), h_ko.to(device)
    d_keys = torch.empty(n_keys, dtype=torch.int64, device=device)
    d_len = torch.empty(len(off) - 1, dtype=torch.int32, device=device)
    h_len = torch.empty(len(off) - 1, dtype=torch.int32).pin_memory()

    def resident():
        GenKeyVectorBatch(d_toks, d_off, bs, d_ko, n_keys, out=d_keys)
        searcher.PrefixMatch(d_keys, d_ko, out=d_len)

    # End to end: tokens start in pinned host memory and the lengths end there.  The hash kernel's time is the
    # latency of the longest chain, not its volume, so cutting the batch into many ranges to overlap copy and
    # compute would repeat that latency per range: one range is fastest at this size (more only pay off when a
    # range's copy takes much longer than the longest chain).
    n_req = len(off) - 1
    n_chunks = 1
    bounds = [int(np.searchsorted(off, off[-1] * c // n_chunks)) for c in range(n_chunks)] + [n_req]
    bounds = sorted(set(min(max(b, 0), n_req) for b in bounds))
    streams = [torch.cuda.Stream(device), torch.cuda.Stream(device)]

    def e2e():
        main = torch.cuda.current_stream(device)
        d_off.copy_(h_off, non_blocking=True)
        d_ko.copy_(h_ko, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record(main)
        for c in range(len(bounds) - 1):
            r0, r1 = bounds[c], bounds[c + 1]
            t0, t1 = int(off[r0]), int(off[r1])
            st = streams[c % 2]
            st.wait_event(ready)
            with torch.cuda.stream(st):
                d_toks[t0:t1].copy_(h_toks[t0:t1], non_blocking=True)
                GenKeyVectorBatch(d_toks, d_off[r0:r1 + 1], bs, d_ko[r0:r1 + 1], n_keys, out=d_keys)
                searcher.PrefixMatch(d_keys, d_ko[r0:r1 + 1], out=d_len[r0:r1])
        for st in streams:
            main.wait_stream(st)
        h_len.copy_(d_len, non_blocking=True)

    out = {}
    for name, fn in (("resident", resident), ("e2e", e2e)):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        out[name] = n_keys * steps / (e0.elapsed_time(e1) * 1e-3)
    matched = int(h_len.sum().item())
    write_cycle = run_write_cycle(device, pkeys, d_keys, d_ko, max(3, steps // 4))
    return dict(write_cycle=write_cycle,
                workload="4096 requests x 512-8192 uint32 tokens, block 64, 50% prefix reuse, index of 200k prior "
                         "blocks; hash + prefix match",
                token_blocks=n_keys, matched_blocks=matched, token_blocks_per_s=out["resident"],
                block_size=bs, longest_request_tokens=int(np.max(off[1:] - off[:-1])),
                e2e_token_blocks_per_s=out["e2e"], h2d_bytes_per_step=int(h_toks.numel() * 4 + h_off.numel() * 16),
                d2h_bytes_per_step=int(h_len.numel() * 4), gpu_launches_per_step=2), (toks, off, ko, bs, ptoks, poff)


def run_write_cycle(device, prior_keys, d_keys, d_ko, reps):
    """The write side of the same batch: StartWriteCache of all requests in one call (filter + new locations in
    CLS_WRITING, answered as if the requests were served in order), then FinishWriteCache of all sessions.  Every
    repetition starts from an index that holds the prior blocks only.  Checked by what must hold afterwards: every
    request's keys are served in full, every key is in the index once, and no request was left a key to write twice."""
    import torch
    from tair_kvcache_b200.manager import BatchMetaSearcher, BlockIndex, encode_locations
    n_req = d_ko.numel() - 1
    start_ms, finish_ms = [], []
    for _ in range(reps):
        index = BlockIndex(prior_keys.numel() + d_keys.numel(), device)
        index.upsert(prior_keys, None, encode_locations([(3, 4)]))
        searcher = BatchMetaSearcher(index)
        torch.cuda.synchronize(device)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        sessions = searcher.StartWriteCache(d_keys, d_ko, 4)
        ev[1].record()
        codes = searcher.FinishWriteCache(sessions, success_off=sessions.new_off[1:] - sessions.new_off[:-1])
        ev[2].record()
        torch.cuda.synchronize(device)
        start_ms.append(ev[0].elapsed_time(ev[1]))
        finish_ms.append(ev[1].elapsed_time(ev[2]))
    new_locations = int(sessions.new_off[-1].item())
    served = searcher.PrefixMatch(d_keys, d_ko)
    distinct = int(torch.unique(torch.cat([prior_keys, d_keys])).numel())
    ok = (bool(torch.equal(served.long(), d_ko[1:] - d_ko[:-1])) and int(codes.abs().sum().item()) == 0 and
          index.stats()[1] == distinct and new_locations == distinct - int(torch.unique(prior_keys).numel()))
    start, finish = float(np.median(start_ms)), float(np.median(finish_ms))
    return {"requests": n_req, "keys": int(d_keys.numel()), "new_locations": new_locations,
            "start_write_ms": start, "finish_write_ms": finish,
            "keys_per_s": d_keys.numel() / ((start + finish) * 1e-3), "gpu_launches": 7, "parity_ok": ok,
            "parity": "after the cycle every request is served in full, the index holds every distinct key once, "
                      "and the sessions hold every new key exactly once"}


def run_prefix_cpu_reference(data, threads, budget_s=12.0):
    """The reference's own CPU path for this configuration, compiled from its sources (oracle/_ref/
    libkvcm_ref_searcher.so): the GenKeyVector loop around hashInt64Array, then MetaSearcher::PrefixMatch over its
    MetaIndexer - per key a look-up in its table and a JSON parse of the key's location map - one request per call
    on `threads` host threads.  Its local meta backend runs without a storage URI (in memory, the reference's own
    switch); with a file it rewrites the file on every mutation and the 200,000-key index would take a day to build.
    Returns (token-blocks/s, repetitions, seconds the index took to build) or None when the library is not there."""
    from oracle import kvcm_oracle as oracle
    from oracle import ref_searcher
    if not ref_searcher.available():
        return None
    toks, off, ko, bs, ptoks, poff = data
    pkeys, _ = oracle.hash_blocks(ptoks, poff, bs, threads=threads)
    pkeys = pkeys[:200000]
    t0 = time.perf_counter()
    searcher = ref_searcher.RefSearcher(max_keys=2 * len(pkeys), in_memory=True)
    for a in range(0, len(pkeys), 20000):
        searcher.add(pkeys[a:a + 20000], 4, oracle.CLS_SERVING)
    built_s = time.perf_counter() - t0
    t64 = np.ascontiguousarray(toks, dtype=np.int64)  # the reference's token ids are int64 (meta_service.proto)
    n, t_total = 0, 0.0
    while t_total < budget_s and n < 20:
        t0 = time.perf_counter()
        searcher.prefix_match_batch(t64, off, bs, threads=threads)
        t_total += time.perf_counter() - t0
        n += 1
    return int(ko[-1]) * n / t_total, n, built_s


def prefix_cpu_baseline(data, threads):
    """cpu_baseline of the prefix-match configuration: the reference itself where its compiled searcher travelled
    with the build, else the oracle's restatement (which leaves out the reference's per-key JSON work)."""
    try:
        ref = run_prefix_cpu_reference(data, threads)
    except (OSError, RuntimeError, AttributeError) as err:  # the library is there but does not load or run here
        print("reference searcher not usable (%s): timing the restatement instead" % err, file=sys.stderr)
        ref = None
    if ref is not None:
        value, n_rep, built_s = ref
        return {"value": value, "unit": "token-blocks/s", "cores": threads, "kind": "reference",
                "sample": "the whole workload, %d repetitions, through the reference's own GenKeyVector + "
                          "MetaSearcher::PrefixMatch compiled from its sources (local meta backend in memory; the "
                          "200,000-key index took %.1f s to build and is not timed)" % (n_rep, built_s)}
    value, n_rep = run_prefix_cpu(data, threads)
    return {"value": value, "unit": "token-blocks/s", "cores": threads, "kind": "port",
            "sample": "the whole workload, %d repetitions; the oracle's restatement, which omits the reference's "
                      "per-key JSON parse and string copies and so over-states the reference" % n_rep}


def run_prefix_cpu(data, threads, budget_s=12.0):
    from oracle import kvcm_oracle as oracle
    toks, off, ko, bs, ptoks, poff = data
    pkeys, _ = oracle.hash_blocks(ptoks, poff, bs, threads=threads)
    ox = oracle.Index()
    ox.put_uniform(pkeys[:200000])
    n, t_total = 0, 0.0
    while t_total < budget_s and n < 20:
        t0 = time.perf_counter()
        keys, ko2 = oracle.hash_blocks(toks, off, bs, threads=threads)
        ox.prefix_match_batch(keys, ko2, threads=threads)
        t_total += time.perf_counter() - t0
        n += 1
    return int(ko[-1]) * n / t_total, n


# ----------------------------------------------------------------------------------------------
# main arms
# ----------------------------------------------------------------------------------------------
def main_reference(args, cfg, rank):
    """CPU arm of the transfer workloads: the same step on the host cores (rank 0 only), `--steps` steps after
    `--warmup` warm-up steps, on as many of the workload's blocks as the host memory holds."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    gbs, ms, sample, n = run_cpu_transfer(cfg, threads, args.steps, args.warmup, budget_s=240.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": transfer_config(cfg, full_payload(cfg)),
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample + "; the reference has no CPU gather/scatter (Triton only), so this arm "
                                            "times the CPU restatement of the same index rule with all host threads"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def measure_link(ctx, d_buf, h_out, h_in, piece=256 << 20, reps=3):
    """What the host link gives plain copies, with no kernel and no operator in the way: every rank, after a
    barrier, copies `d_buf` to the pinned `h_out` and the pinned `h_in` to `d_buf`'s second half with
    cudaMemcpyAsync in pieces of 256 MiB - each direction alone, then both at once on two streams - and the
    slowest rank counts.  GB/s of payload per direction and per GPU."""
    import torch
    n = min(d_buf.numel() // 2, h_out.numel(), h_in.numel())
    s_out, s_in = torch.cuda.Stream(ctx.device), torch.cuda.Stream(ctx.device)
    d_src, d_dst = d_buf[:n], d_buf[n:2 * n]

    def run(out, inn):
        for a in range(0, n, piece):
            b = min(n, a + piece)
            if out:
                with torch.cuda.stream(s_out):
                    h_out[a:b].copy_(d_src[a:b], non_blocking=True)
            if inn:
                with torch.cuda.stream(s_in):
                    d_dst[a:b].copy_(h_in[a:b], non_blocking=True)

    res = {}
    for name, out, inn in (("d2h_alone", True, False), ("h2d_alone", False, True), ("both", True, True)):
        run(out, inn)
        torch.cuda.synchronize(ctx.device)
        ctx.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            run(out, inn)
        torch.cuda.synchronize(ctx.device)
        dt = ctx.max_over_ranks([time.perf_counter() - t0])[0]
        res[name] = n * h_out.element_size() * reps / dt / 1e9
    return res


def run_transfer(args, cfg, ctx, with_e2e=True, with_cpu=True):
    """One transfer workload on this rank's GPU (every rank its own tensor-parallel slice); returns the JSON line
    on every rank (the figures are already reduced over the ranks)."""
    import torch

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200.kernel import (batch_gather_kv_caches, batch_gather_kv_pages, batch_scatter_kv_caches,
                                          batch_scatter_kv_pages)

    rank, world, device = ctx.rank, ctx.world, ctx.device
    w = build_transfer_workload(cfg, device, seed=0xB2000002 + rank)
    ptrs, table, slots, staging = w["ptrs"], w["table"], w["slots"], w["staging"]
    ppb, page_bytes, pool_pages, payload = w["ppb"], w["page_bytes"], w["pool_pages"], w["payload"]

    def gather():
        batch_gather_kv_pages(ptrs, staging, table, slots, ppb, page_bytes, pool_pages)

    def scatter():
        batch_scatter_kv_pages(ptrs, staging, table, slots, ppb, page_bytes, pool_pages)

    gather()
    torch.cuda.synchronize(device)
    gather_ok = verify_gather(w)

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()  # before the warm-up, so the GPU does not idle between warm-up and the timed region
    for _ in range(args.warmup):
        gather()
        scatter()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    ctx.barrier()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_begin()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(args.steps):
        ev[k][0].record()
        gather()
        ev[k][1].record()
        scatter()
        ev[k][2].record()
    stop.record()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_end()
    ctx.barrier()
    clocks = sampler.stop() if sampler else None
    elapsed_ms = start.elapsed_time(stop)
    gather_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    scatter_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    elapsed_ms, gather_ms, scatter_ms = ctx.max_over_ranks([elapsed_ms, gather_ms, scatter_ms])
    alg_bytes_step = 4 * payload  # gather: read + write payload; scatter: the same
    value = world * alg_bytes_step * args.steps / (elapsed_ms * 1e-3) / 1e9
    scatter_ok = verify_scatter(w, scatter)

    # ---- end to end: pinned host staging through the operator API, python index lists included.
    # As in the reference connector (kv_cache_manager/py_connector/vllm/data_transfer.py:77-78,138,203) saves run
    # on one CUDA stream and loads on another, each with its own pool of pinned staging blocks, so the two PCIe
    # directions work at the same time.  A step = every save task (gather -> host) and every load task
    # (host -> scatter) once.
    T = ppb * cfg["page_tokens"]
    task_blocks = min(128, w["n_blocks"])  # blocks per save / load task of the reference connector
    n_tasks = min(w["n_blocks"] // task_blocks, 8)
    dim = cfg["token_bytes"] // 2
    task_payload = task_blocks * w["n_pools"] * T * cfg["token_bytes"]
    idx_bytes = n_tasks * 2 * (task_blocks * T + task_blocks) * 4
    e2e = None
    if with_e2e:
        save_pool = torch.empty(task_blocks, w["n_pools"], T, dim, dtype=torch.bfloat16, pin_memory=True)
        load_pool = torch.empty(n_tasks, task_blocks, w["n_pools"], T, dim, dtype=torch.bfloat16, pin_memory=True)
        table_np = table.cpu().numpy().reshape(w["n_blocks"], ppb)
        tok_np = (table_np[:, :, None].astype(np.int64) * cfg["page_tokens"] +
                  np.arange(cfg["page_tokens"])[None, None, :]).reshape(w["n_blocks"], T)
        task_tok = [tok_np[i * task_blocks:(i + 1) * task_blocks].reshape(-1).tolist() for i in range(n_tasks)]
        task_slots = list(range(task_blocks))

        def torch_gather_of_task(i):
            """What storage hands back for task i: the blocks as a torch gather of the pools lays them out
            ([block, pool, tokens x dim]); built without the kernels under test."""
            pages = torch.from_numpy(table_np[i * task_blocks:(i + 1) * task_blocks]).to(device).long()
            return torch.stack([pool.view(pool_pages, -1)[pages].reshape(task_blocks, -1) for pool in w["pools"]], 1)

        for i in range(n_tasks):
            load_pool[i].view(torch.int32).view(task_blocks, w["n_pools"], -1).copy_(torch_gather_of_task(i))
        torch.cuda.synchronize(device)
        save_stream, load_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)

        def e2e_step():
            for i in range(n_tasks):
                with torch.cuda.stream(save_stream):
                    batch_gather_kv_caches(ptrs, save_pool, task_tok[i], task_slots, T, dim)
                with torch.cuda.stream(load_stream):
                    batch_scatter_kv_caches(ptrs, load_pool[i], task_tok[i], task_slots, T, dim)

        e2e_steps = max(1, min(args.steps, 3))
        e2e_step()
        torch.cuda.synchronize(device)
        ctx.barrier()
        t_wall = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize(device)  # both streams drained: every staged byte has crossed PCIe
        e2e_ms = (time.perf_counter() - t_wall) * 1e3  # wall clock around the calls: host list conversion counts
        e2e_ms = ctx.max_over_ranks([e2e_ms])[0]
        e2e_value = world * 4 * task_payload * n_tasks * e2e_steps / (e2e_ms * 1e-3) / 1e9
        # parity of both directions, against torch indexing.  Save: the pinned blocks of the last save task.  Load:
        # one task scattered from pinned host memory into zeroed scratch pools through a page table of its own,
        # then every scratch page compared with the page of the real pools it stands for.
        want_last = torch_gather_of_task(n_tasks - 1)
        save_ok = bool(torch.equal(save_pool.view(torch.int32).view(task_blocks, w["n_pools"], -1).to(device),
                                   want_last))
        del want_last
        n_scr = task_blocks * ppb
        scratch = [torch.zeros(n_scr * page_bytes // 4, dtype=torch.int32, device=device) for _ in range(w["n_pools"])]
        scr_ptrs = torch.tensor([t.data_ptr() for t in scratch], dtype=torch.int64, device=device)
        scr_table = np.random.default_rng(5).permutation(n_scr).reshape(task_blocks, ppb)
        scr_tok = (scr_table[:, :, None].astype(np.int64) * cfg["page_tokens"] +
                   np.arange(cfg["page_tokens"])[None, None, :]).reshape(-1).tolist()
        batch_scatter_kv_caches(scr_ptrs, load_pool[0], scr_tok, task_slots, T, dim)
        torch.cuda.synchronize(device)
        real = torch.from_numpy(table_np[:task_blocks]).to(device).long()
        scr = torch.from_numpy(scr_table).to(device).long()
        load_ok = all(bool(torch.equal(sp.view(n_scr, -1)[scr], pool.view(pool_pages, -1)[real]))
                      for sp, pool in zip(scratch, w["pools"]))
        # the host link's own ceiling, measured beside it with plain copies of the same pinned pools
        del scratch
        d_buf = torch.empty(2 * save_pool.numel(), dtype=torch.int16, device=device)
        link = measure_link(ctx, d_buf, save_pool.view(torch.int16).view(-1),
                            load_pool[0].view(torch.int16).view(-1))
        per_dir = e2e_value / 4 / world  # payload GB/s per direction and GPU through the operators
        e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": task_payload * n_tasks + idx_bytes,
               "d2h_bytes_per_step": task_payload * n_tasks, "parity_ok": save_ok and load_ok,
               "parity": {"saved_blocks_equal_torch_gather": save_ok, "load_into_zeroed_scratch_pools": load_ok},
               "payload_GBps_per_direction_per_gpu": per_dir,
               "link_peak": {"unit": "GB/s of payload per direction per GPU, plain cudaMemcpyAsync of the same pinned "
                                     "pools in 256 MiB pieces, max over ranks",
                             "both_directions_at_once": link["both"], "d2h_alone": link["d2h_alone"],
                             "h2d_alone": link["h2d_alone"], "aggregate_both": link["both"] * world},
               "frac_of_link": per_dir / link["both"],
               "note": "%d save tasks and %d load tasks of %d blocks per step on two streams, staging in pinned "
                       "host memory, token-index lists converted per call" % (n_tasks, n_tasks, task_blocks)}
        del save_pool, load_pool, d_buf

    peak, peak_kind = peaks()
    gather_gbs = 2 * payload / (gather_ms * 1e-3) / 1e9
    scatter_gbs = 2 * payload / (scatter_ms * 1e-3) / 1e9
    config = transfer_config(cfg, payload)
    config["pool_pages"] = pool_pages
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic", "config": config,
        "parity_sample_ok": gather_ok and scatter_ok,
        "parity": {"gather_all_tiles_equal_torch_gather": gather_ok,
                   "scatter_of_changed_staging_all_pages_and_untouched_sample": scatter_ok},
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "MoveRowsBulkKernel<gather>", "achieved": gather_gbs, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": gather_gbs / peak,
                     "traffic": int(DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * 2 * payload),
                     "traffic_source": "ncu capture on a reduced case scaled by blocks moved",
                     "algorithmic_bytes_per_launch": 2 * payload, "launch_ms": gather_ms,
                     "scatter": {"kernel": "MoveRowsBulkKernel<scatter>", "achieved": scatter_gbs,
                                 "frac": scatter_gbs / peak, "launch_ms": scatter_ms}},
        "gpu_launches": 2 * args.steps * world,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and with_cpu and not args.no_cpu:
        threads = os.cpu_count() or 1
        cpu_gbs, _, sample, _ = run_cpu_transfer(cfg, threads, 40, 1, budget_s=8.0, max_payload=2 << 30)
        line["cpu_baseline"] = {"value": cpu_gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
    return line


def extra_of(line, keep=("metric", "value", "unit", "ms_per_step", "steps", "warmup", "scaling", "config",
                         "parity_sample_ok", "parity", "roofline", "clocks", "gpu_launches", "e2e", "cpu_baseline")):
    """A workload's line cut down to what an extra key of the default line carries."""
    return {k: line[k] for k in keep if k in line}


def main_prefix(args, ctx):
    """--workload c1: the CPU-runnable prefix-match configuration on its own (hash + prefix match of 4,096
    requests against an index of 200k prior blocks).  Replicas only: every rank would run the same batch, so
    rank 0 alone runs it.  `ctx` is None for the CPU arm."""
    if ctx is not None and ctx.rank != 0:
        return
    threads = os.cpu_count() or 1
    if args.impl == "reference":
        data = build_prefix_workload()
        (ptoks, poff), (toks, off), _, bs = data
        from oracle import kvcm_oracle as oracle
        base = prefix_cpu_baseline((toks, off, oracle.key_offsets(off, bs), bs, ptoks, poff), threads)
        cpu = base["value"]
        print(json.dumps({"impl": "reference", "metric": "prefix_match_token_blocks_per_s", "value": cpu,
                          "unit": "token-blocks/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": 0,
                          "higher_is_better": True, "dtype": "int64", "data": "synthetic",
                          "config": {"workload": "4096 requests x 512-8192 uint32 tokens, block 64, 50% prefix reuse, "
                                                 "index of 200k prior blocks; hash + prefix match"},
                          "cpu_baseline": base,
                          "e2e": {"value": cpu, "unit": "token-blocks/s", "h2d_bytes_per_step": 0,
                                  "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return
    import tair_kvcache_b200  # noqa: F401
    device = ctx.device
    pm, data = run_prefix_gpu(device, args.steps, args.warmup)
    line = {"metric": "prefix_match_token_blocks_per_s", "value": pm["token_blocks_per_s"], "unit": "token-blocks/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * pm["token_blocks"] / pm["token_blocks_per_s"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": {"workload": pm["workload"]},
            "e2e": {"value": pm["e2e_token_blocks_per_s"], "unit": "token-blocks/s",
                    "h2d_bytes_per_step": pm["h2d_bytes_per_step"], "d2h_bytes_per_step": pm["d2h_bytes_per_step"]},
            "gpu_launches": 2 * args.steps}
    # Roofline of the step (hash + match kernels together): algorithmic bytes per token block = the block's tokens
    # + the key written + one index slot read.  The binding limit is the dependent chain of the longest request
    # (~40 cycles per token), stated beside the HBM fraction.
    peak, peak_kind = peaks()
    ms_step = 1e3 * pm["token_blocks"] / pm["token_blocks_per_s"]
    achieved = pm["token_blocks"] * (4 * pm["block_size"] + 8 + 16) / (ms_step * 1e-3) / 1e9
    line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "traffic": None, "peak_kind": peak_kind,
                        "chain_latency_floor_ms": pm["longest_request_tokens"] * 40 / 1.965e6}
    line["write_cycle"] = pm["write_cycle"]
    if not args.no_cpu:
        line["cpu_baseline"] = prefix_cpu_baseline(data, threads)
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# sliding-window + prefix match at scale, index sharded by hash range (--workload c4)
# ----------------------------------------------------------------------------------------------
def build_window_workload(device, rank, world, n_req_total, n_roots, index_keys_total, seed=0xB2000004, bs=16,
                          min_len=256, max_len=131072):
    """This rank's share of: n_req_total requests with log-uniform lengths in [min_len, max_len], each sharing a
    random-length prefix of one of n_roots root prompts chosen by Zipf(1.1); index content = the blocks of the root
    prompts (for 30 % of them only a trailing multiple of 256 blocks, as a sliding-window cache would retain) plus
    the blocks of the first requests, index_keys_total keys in all.  Every rank derives the same global picture
    from the seed and materialises only its own slice.  Tokens are generated on the GPU."""
    import torch
    rng = np.random.default_rng(seed)

    def loguniform(n):
        return np.exp(rng.uniform(np.log(min_len), np.log(max_len), size=n)).astype(np.int64)

    root_len = loguniform(n_roots)
    req_len = loguniform(n_req_total)
    zipf = 1.0 / np.arange(1, n_roots + 1) ** 1.1
    root_of = rng.choice(n_roots, size=n_req_total, p=zipf / zipf.sum())
    share = (rng.random(n_req_total) * (np.minimum(req_len, root_len[root_of]) + 1)).astype(np.int64)
    keep_tail = rng.random(n_roots) < 0.3  # roots of which only a trailing window multiple is indexed
    tail_windows = rng.integers(1, 4, size=n_roots)

    gen = torch.Generator(device=device).manual_seed(seed)  # same stream on every rank: same root tokens
    root_off = np.zeros(n_roots + 1, dtype=np.int64)
    np.cumsum(root_len, out=root_off[1:])
    roots = torch.randint(0, 151936, (int(root_off[-1]),), dtype=torch.int32, device=device, generator=gen)

    mine = np.arange(rank, n_req_total, world)  # round-robin: lengths are i.i.d., shares balance
    my_len = req_len[mine]
    off = np.zeros(len(mine) + 1, dtype=np.int64)
    np.cumsum(my_len, out=off[1:])
    gen_r = torch.Generator(device=device).manual_seed(seed + 1 + rank)
    toks = torch.randint(0, 151936, (int(off[-1]),), dtype=torch.int32, device=device, generator=gen_r)
    for j, r in enumerate(mine):
        m = int(share[r])
        if m:
            a, b = int(off[j]), int(root_off[root_of[r]])
            toks[a:a + m] = roots[b:b + m]
    return dict(roots=roots, root_off=root_off, keep_tail=keep_tail, tail_windows=tail_windows, toks=toks, off=off,
                mine=mine, bs=bs, index_keys_total=index_keys_total, req_len=req_len)


def run_window(args, ctx):
    """--workload c4 (and the `window_match` key of the default line): hash + prefix match + sliding-window match
    of this rank's share of the requests against the index split by hash range over the ranks.  Returns the JSON
    line on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200.manager import (BatchMetaSearcher, CudaShardBackend, GenKeyVectorBatch,
                                           ShardedMetaSearcher, encode_locations, key_offsets, length_order)

    rank, world, device = ctx.rank, ctx.world, ctx.device
    n_req_total = args.n_requests or 65536
    index_keys = args.index_keys or 10_000_000
    sw = 4096 // 16
    w = build_window_workload(device, rank, world, n_req_total, 1000, index_keys)
    bs = w["bs"]
    word = encode_locations([(3, 4)])

    def hash_csr(tokens, off_np):
        ko = key_offsets(off_np, bs)
        order, cap = length_order(off_np, with_residency=True)
        keys = GenKeyVectorBatch(tokens, torch.from_numpy(off_np).to(device), bs, torch.from_numpy(ko).to(device),
                                 int(ko[-1]), order=torch.from_numpy(order).to(device), warps_per_sm=cap)
        return keys, ko

    # ---- index content: root blocks (this rank hashes a slice of the roots), then request blocks up to the quota
    backend = CudaShardBackend(2 * index_keys // world + 1024, device)
    searcher = None
    if world > 1:  # exchange areas of the peer-memory route: one per stream, room for a rank's whole batch + 25 %
        searcher = ShardedMetaSearcher(backend, mode=args.shard_mode, route_areas=2,
                                       route_capacity=int(key_offsets(w["off"], bs)[-1] * 1.25) + 65536)
    local_index = BatchMetaSearcher(backend.index)

    def insert(keys):
        if world > 1:
            searcher.upsert(keys, word)
        else:
            backend.upsert_owned(keys, word, 1, 0)

    root_keys, root_ko = hash_csr(w["roots"], w["root_off"])
    keep = torch.ones(root_keys.numel(), dtype=torch.bool, device=device)
    for r in np.nonzero(w["keep_tail"])[0]:
        a, b = int(root_ko[r]), int(root_ko[r + 1])
        tail = min(b - a, int(w["tail_windows"][r]) * sw)
        keep[a:b - tail] = False
    my_roots = torch.zeros_like(keep)
    for r in range(rank, len(w["root_off"]) - 1, world):
        my_roots[int(root_ko[r]):int(root_ko[r + 1])] = True
    insert(root_keys[keep & my_roots].contiguous())
    n_root_keys = int(keep.sum().item())
    req_keys, req_ko = hash_csr(w["toks"], w["off"])
    quota = max(0, index_keys - n_root_keys) // world  # each rank contributes the blocks of its first requests
    n_from_reqs = int(np.searchsorted(req_ko, quota, side="right")) - 1
    insert(req_keys[:int(req_ko[n_from_reqs])].contiguous())
    torch.cuda.synchronize(device)
    stored = backend.index.stats()[1]

    d_off = torch.from_numpy(w["off"]).to(device)
    d_ko = torch.from_numpy(req_ko).to(device)
    n_keys = int(req_ko[-1])
    d_keys = torch.empty(max(n_keys, 1), dtype=torch.int64, device=device)
    order_np, residency = length_order(w["off"], with_residency=True)  # ragged lengths: longest chains first
    d_order = torch.from_numpy(order_np).to(device)

    def step_serial():
        keys = GenKeyVectorBatch(w["toks"], d_off, bs, d_ko, n_keys, out=d_keys, order=d_order, warps_per_sm=residency)
        if world > 1 and args.shard_mode == "peer":  # every key is probed at its owner over NVLink: no collective
            return searcher.PrefixMatch(keys, d_ko), searcher.ReverseRollSlideWindowMatch(keys, d_ko, sw)
        if world > 1 and args.shard_mode in ("route", "route_peer"):  # keys to their owners, one flag byte back, both queries local
            r = searcher.Route(keys, d_ko)
            return searcher.PrefixMatch(r), searcher.ReverseRollSlideWindowMatch(r, sw_size=sw)
        if world > 1:
            g = searcher.Gather(keys, d_ko)  # one exchange of the keys serves both queries
            return searcher.PrefixMatch(g), searcher.ReverseRollSlideWindowMatch(g, sw_size=sw)
        return local_index.PrefixMatch(keys, d_ko), local_index.ReverseRollSlideWindowMatch(keys, d_ko, sw)

    # The step is ruled by the dependent chains of the few longest requests (131k tokens = 2.6 ms), during which
    # most SMs idle.  So the batch is laid out longest first (a batcher is free to order its requests) and cut in two:
    # the long head is hashed and matched on one stream while the rest is hashed and matched on another.  Same
    # kernels, same results per request.
    routed = args.shard_mode in ("route", "route_peer")
    overlap = not args.no_overlap and (world == 1 or args.shard_mode == "peer" or routed)
    if overlap:
        my_len = w["off"][1:] - w["off"][:-1]
        perm = np.argsort(-my_len, kind="stable")  # sorted position -> request
        off_s = np.zeros(len(perm) + 1, dtype=np.int64)
        np.cumsum(my_len[perm], out=off_s[1:])
        toks_s = torch.empty_like(w["toks"])
        for pos, j in enumerate(perm):
            toks_s[int(off_s[pos]):int(off_s[pos + 1])] = w["toks"][int(w["off"][j]):int(w["off"][j + 1])]
        ko_s = key_offsets(off_s, bs)
        d_off_s, d_ko_s = torch.from_numpy(off_s).to(device), torch.from_numpy(ko_s).to(device)
        if args.long_fraction is None:
            # measured: one GPU, head at 2 warps per SM: 0.3 / 0.5 / 0.7 -> 3.17 / 3.68 / 3.73 ms per step;
            # 2 GPUs routed, head at 4: 0.5 / 0.7 -> 2.80 / 2.84 ms
            args.long_fraction = "0.7" if world > 1 and routed else "0.3"
        if args.head_cap is None:  # one GPU: head 4 / 2 warps per SM -> 3.27 / 3.17 ms; 2 GPUs routed: 2.84 / 2.99 ms
            args.head_cap = "4" if world > 1 and routed else "2"
        # several thresholds (comma-separated) cut the head into length classes, longest first, each with its own
        # stream and cap, so that the keys of a class are matched while the longer chains before it still run;
        # measured on one GPU: 0.85,0.3 / 0.7,0.3 / 0.6,0.3 -> 4.34 / 3.72 / 3.43 ms per step against 3.21 for 0.3
        # alone - the step is close to the sum of the kernels' throughput-bound times, more launches only crowd it
        fractions = sorted((float(f) for f in str(args.long_fraction).split(",")), reverse=True)
        caps = [int(c) for c in str(args.head_cap).split(",")]
        caps += [caps[-1]] * (len(fractions) - len(caps))
        if world > 1 and routed and len(fractions) > 1:
            raise SystemExit("the routed shard modes take one --long-fraction")
        edges_long = [int(np.count_nonzero(my_len >= f * my_len.max())) for f in fractions]
        n_long = edges_long[-1]
        prefix_s = torch.empty(len(perm), dtype=torch.int32, device=device)
        window_s = torch.empty(len(perm), dtype=torch.int32, device=device)
        inv = torch.from_numpy(np.argsort(perm)).to(device)  # request -> sorted position
        # (first request, end, hashing warps per SM): 4 for the head, so that its chains sit alone on their
        # schedulers, and 3 for the rest, which then shares an SM with a head warp without crowding its scheduler
        # (measured: rest at 2 / 3 / 4 / unlimited warps per SM -> 4.12 / 3.98 / 4.29 / 4.25 ms per step)
        parts = [(a, b, c) for a, b, c in zip([0] + edges_long[:-1], edges_long, caps)] + \
                [(n_long, len(perm), args.rest_cap)]
        if not (world > 1 and routed) and args.rest_chunks > 1 and len(perm) - n_long > args.rest_chunks:
            # The rest is bound by throughput, and its two halves use different resources: hashing the integer
            # pipe, matching the random-sector rate of the memory system.  Cut into chunks of equal token count on
            # streams of their own, the match of one chunk runs under the hash of the next.
            cuts = np.searchsorted(off_s, off_s[n_long] + (off_s[-1] - off_s[n_long]) *
                                   np.arange(1, args.rest_chunks) // args.rest_chunks)
            edges = sorted(set([n_long] + [int(c) for c in cuts if n_long < c < len(perm)] + [len(perm)]))
            parts = parts[:-1] + [(a, b, args.rest_cap) for a, b in zip(edges[:-1], edges[1:])]
        # the head's stream comes first in the queues of the SMs: once its long chains are through, its matchers
        # are not left waiting behind the kernels of the rest
        streams = [torch.cuda.Stream(device, priority=-1 if i < len(fractions) and args.head_priority else 0)
                   for i in range(len(parts))]
        flag_bytes = torch.empty(max(n_keys, 1), dtype=torch.uint8, device=device)
        match = searcher if world > 1 else local_index
        # the keys of a part as a batch of its own (routing sends whole batches)
        rel_ko = [(d_ko_s[a:b + 1] - int(ko_s[a])).contiguous() for a, b, _ in parts]

    def step_overlapped_routed(marks=None):
        """Both parts are hashed at once; the short requests are routed and matched while the long chains still
        run, then the long ones.  Every rank issues the collectives in the same order (rest, then head), parts
        without requests included."""
        def mark(label, stream):
            if marks is not None:
                marks.append((label, torch.cuda.Event(enable_timing=True)))
                marks[-1][1].record(stream)

        main = torch.cuda.current_stream(device)
        start = torch.cuda.Event()
        start.record(main)
        mark("start", main)
        for name, st, (a, b, cap) in zip(("head", "rest"), streams, parts):
            st.wait_event(start)
            if b > a:
                with torch.cuda.stream(st):
                    GenKeyVectorBatch(toks_s, d_off_s[a:b + 1], bs, d_ko_s[a:b + 1], n_keys, out=d_keys,
                                      warps_per_sm=cap)
            mark(name + "_hashed", st)
        for which in (1, 0):
            a, b, _ = parts[which]
            with torch.cuda.stream(streams[which]):
                r = searcher.Route(d_keys[int(ko_s[a]):int(ko_s[b])], rel_ko[which], area=which)
                mark(("head", "rest")[which] + "_routed", streams[which])
                prefix_s[a:b] = searcher.PrefixMatch(r)
                window_s[a:b] = searcher.ReverseRollSlideWindowMatch(r, sw_size=sw)
                mark(("head", "rest")[which] + "_matched", streams[which])
            main.wait_stream(streams[which])
        return prefix_s[inv], window_s[inv]

    def step_overlapped(marks=None):
        main = torch.cuda.current_stream(device)
        start = torch.cuda.Event(enable_timing=marks is not None)
        start.record(main)
        if marks is not None:
            marks.append(("start", start))
        for i, (st, (a, b, cap)) in enumerate(zip(streams, parts)):
            if b <= a:
                continue
            st.wait_event(start)
            with torch.cuda.stream(st):
                GenKeyVectorBatch(toks_s, d_off_s[a:b + 1], bs, d_ko_s[a:b + 1], n_keys, out=d_keys, warps_per_sm=cap)
                if marks is not None:
                    marks.append(("part%d_hashed" % i, torch.cuda.Event(enable_timing=True)))
                    marks[-1][1].record(st)
                if world == 1 and args.match_via == "flags":
                    # one look-up per key serves both questions
                    ka, kb = int(ko_s[a]), int(ko_s[b])
                    fl = local_index.BatchGet(d_keys[ka:kb], out=flag_bytes[ka:kb])
                    local_index.PrefixMatchFromFlags(fl, rel_ko[i], out=prefix_s[a:b])
                    local_index.ReverseRollSlideWindowMatchFromFlags(fl, rel_ko[i], sw, out=window_s[a:b])
                else:
                    prefix_s[a:b] = match.PrefixMatch(d_keys, d_ko_s[a:b + 1])
                    window_s[a:b] = match.ReverseRollSlideWindowMatch(d_keys, d_ko_s[a:b + 1], sw)
                if marks is not None:
                    marks.append(("part%d_matched" % i, torch.cuda.Event(enable_timing=True)))
                    marks[-1][1].record(st)
            main.wait_stream(st)
        return prefix_s[inv], window_s[inv]  # back in request order

    step = step_serial
    if overlap:
        step = step_overlapped_routed if world > 1 and routed else step_overlapped

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(args.warmup):
        prefix, window = step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        prefix, window = step()
    e1.record()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_end()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    ms = e0.elapsed_time(e1)
    # where a step goes (one extra untimed step, phases bracketed by events)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    keys = GenKeyVectorBatch(w["toks"], d_off, bs, d_ko, n_keys, out=d_keys, order=d_order, warps_per_sm=residency)
    ev[1].record()
    if world > 1 and routed:
        flags = searcher.Route(keys, d_ko)
        ev[2].record()
        searcher.PrefixMatch(flags)
        searcher.ReverseRollSlideWindowMatch(flags, sw_size=sw)
    elif world > 1:
        searcher.PrefixMatch(keys, d_ko)
        ev[2].record()
        searcher.ReverseRollSlideWindowMatch(keys, d_ko, sw)
    else:
        local_index.PrefixMatch(keys, d_ko)
        ev[2].record()
        local_index.ReverseRollSlideWindowMatch(keys, d_ko, sw)
    ev[3].record()
    torch.cuda.synchronize(device)
    phase_ms = {"hash": ev[0].elapsed_time(ev[1]), "prefix_match": ev[1].elapsed_time(ev[2]),
                "window_match": ev[2].elapsed_time(ev[3])}
    if step is step_overlapped_routed or step is step_overlapped:  # when each part finished, from the step's start
        marks = []
        step(marks)
        torch.cuda.synchronize(device)
        phase_ms["two_stream_timeline"] = {k: round(marks[0][1].elapsed_time(e), 3) for k, e in marks[1:]}
    if world > 1 and routed:
        phase_ms = {"hash": phase_ms["hash"], "dispatch_lookup_combine": phase_ms["prefix_match"],
                    "prefix_and_window_from_flags": phase_ms["window_match"],
                    **{k: v for k, v in phase_ms.items() if k == "two_stream_timeline"}}
    if world == 1:
        # the other index operators on the same keys, outside the timed step: BatchGet (one flag byte per key),
        # FilterWriteCache (what StartWriteCache asks before a write) and the write side (upsert of fresh keys into
        # a second index of the same size, then their erase)
        from tair_kvcache_b200.manager import BlockIndex
        ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        fresh = BlockIndex(max(int(stored), 1024), device)
        some = keys[:min(n_keys, int(stored))]
        local_index.BatchGet(keys)  # untimed first calls: the output tensors come from torch's caching allocator
        local_index.FilterWriteCache(keys, d_ko)
        ev2[0].record()
        local_index.BatchGet(keys)
        ev2[1].record()
        local_index.FilterWriteCache(keys, d_ko)
        ev2[2].record()
        fresh.upsert(some, None, word)
        ev2[3].record()
        fresh.erase(some)
        ev2[4].record()
        torch.cuda.synchronize(device)
        phase_ms.update({"batch_get_all_keys": ev2[0].elapsed_time(ev2[1]),
                         "filter_write_all_requests": ev2[1].elapsed_time(ev2[2]),
                         "upsert_%d_keys" % some.numel(): ev2[2].elapsed_time(ev2[3]),
                         "erase_%d_keys" % some.numel(): ev2[3].elapsed_time(ev2[4])})
        del fresh
    stats = torch.tensor([ms, float(n_keys), float(stored), float((prefix > 0).sum()), float((window >= 0).sum())],
                         dtype=torch.float64, device=device)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        stats[0] = mx[0]
    ms, total_keys, total_stored, n_prefix_hits, n_windows = stats.tolist()

    # ---- parity on a sample of rank 0's requests against the CPU oracle's UNSHARDED index, rebuilt on the CPU from
    # the keys every rank inserted (the root blocks are known to every rank; the request blocks are collected)
    parity = None
    if not args.no_cpu:
        n_ins = int(req_ko[n_from_reqs])
        inserted = [req_keys[:n_ins]]
        if world > 1:
            sizes = torch.zeros(world, dtype=torch.int64, device=device)
            sizes[rank] = n_ins
            dist.all_reduce(sizes)
            width = int(sizes.max().item())
            mine_padded = torch.zeros(max(width, 1), dtype=torch.int64, device=device)
            mine_padded[:n_ins] = req_keys[:n_ins]
            parts_all = [torch.empty_like(mine_padded) for _ in range(world)]
            dist.all_gather(parts_all, mine_padded)
            inserted = [t[:int(n)] for t, n in zip(parts_all, sizes.tolist())]
        if rank == 0:
            from oracle import kvcm_oracle as oracle
            ox = oracle.Index()
            ox.put_uniform(root_keys[keep].cpu().numpy())
            for t in inserted:
                ox.put_uniform(t.cpu().numpy())
            sample = np.random.default_rng(0).choice(len(w["mine"]), size=min(1024, len(w["mine"])), replace=False)
            toks_h = w["toks"].cpu().numpy().view(np.uint32)
            prefix_h, window_h = prefix.cpu().numpy(), window.cpu().numpy()
            parity = True
            for j in sample:
                k = oracle.gen_key_vector(toks_h[w["off"][j]:w["off"][j + 1]], bs)
                ok_keys = np.array_equal(k, req_keys[int(req_ko[j]):int(req_ko[j + 1])].cpu().numpy())
                ec, base = ox.sw_match(k, sw)
                want_w = base if ec == 0 else -2
                parity = bool(parity and ok_keys and ox.prefix_match(k) == int(prefix_h[j]) and
                              want_w == int(window_h[j]))
        del inserted

    if rank == 0:
        longest = int(w["req_len"].max())
        line = {"metric": "prefix_and_window_match_token_blocks_per_s", "value": total_keys * args.steps / (ms * 1e-3),
                "unit": "token-blocks/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int64", "data": "synthetic",
                "config": {"workload": "%d requests, lengths log-uniform 256-131072 tokens, block 16, Zipf(1.1) prefix "
                                       "sharing over 1000 roots, window 256 blocks, index of %d keys split by hash "
                                       "range over %d GPU(s)%s; hash + prefix match + sliding-window match per step"
                                       % (n_req_total, int(total_stored), world,
                                          "" if world == 1 else {
                                              "peer": ", shards probed over NVLink peer loads",
                                              "route": ", keys sent to their owners and one flag byte back "
                                                       "(two all-to-alls per step)",
                                              "route_peer": ", keys stored into their owners' inboxes and one flag "
                                                            "byte stored back over NVLink peer memory",
                                              "exchange": ", all-gather of keys + min/max all-reduce",
                                          }[args.shard_mode]),
                           "token_blocks": int(total_keys), "longest_request_tokens": longest,
                           "requests_with_prefix_hit": int(n_prefix_hits), "requests_with_window": int(n_windows),
                           "shard_mode": args.shard_mode if world > 1 else "one unsharded index",
                           "lookups_per_s": 2 * total_keys * args.steps / (ms * 1e-3),
                           "parity_sample_ok": parity, "phase_ms_rank0": phase_ms,
                           "schedule": ("%d streams: the %d longest requests of rank 0 (length classes >= %s of the "
                                        "longest, %s hashing warps per SM) hashed and matched beside the rest%s%s; "
                                        "phase_ms are the kernels run alone on the whole batch"
                                        % (len(parts), n_long, "/".join("%.2f" % f for f in fractions),
                                           "/".join(str(c) for c in caps[:len(fractions)]),
                                           " (in %d chunks of equal token count)" % (len(parts) - len(fractions))
                                           if len(parts) > len(fractions) + 1 else "",
                                           "; one BatchGet per key feeds both matchers"
                                           if world == 1 and args.match_via == "flags" else ""))
                           if overlap else "one stream"},
                "gpu_launches": ({"peer": 6, "route": 14, "route_peer": 14}[args.shard_mode] if overlap and world > 1
                                 else 3 * len(parts) if overlap else 3 if world == 1 else 7 if routed else 4)
                * args.steps * world}
        # Roofline of the step.  Algorithmic bytes per token block: its 16 tokens (64 B), the key written (8 B), and
        # per matcher the key read (8 B) and one index slot (16 B) = 120 B.  The binding limit is not HBM but the
        # dependent chain of the longest request, one hash step per token: its floor is stated beside the fraction.
        peak, peak_kind = peaks()
        per_gpu = total_keys * 120 / world / (ms / args.steps * 1e-3) / 1e9
        mhz = (clocks or {}).get("sm_mhz") or 1965.0
        line["parity_sample_ok"] = parity
        line["clocks"] = clocks
        line["roofline"] = {
            "bound": "hbm", "kernel": "HashBlocksKernel + matchers (whole step)", "achieved": per_gpu, "peak": peak,
            "peak_kind": peak_kind, "unit": "GB/s", "frac": per_gpu / peak, "traffic": None,
            "algorithmic_bytes_per_token_block": 120,
            "hash_launch_ms_whole_batch": phase_ms["hash"],
            "hash_cycles_per_token_on_longest_chain": phase_ms["hash"] * 1e-3 * mhz * 1e6 / longest,
            "chain_latency_floor_ms": phase_ms["hash"],
            "note": "latency-bound: the hash of the longest request (%d tokens, one dependent step per token) takes "
                    "%.2f ms whatever the number of GPUs; the HBM fraction is reported for completeness" % (
                        longest, phase_ms["hash"])}
    if world > 1:
        if args.shard_mode == "peer":
            searcher.detach_peers()
        if args.shard_mode == "route_peer":
            searcher.detach_route_areas()
    return line if rank == 0 else None


# ----------------------------------------------------------------------------------------------
# mixed trace replay (--workload c5): hash -> replay against all earlier requests -> gather the misses (MLA layout)
# ----------------------------------------------------------------------------------------------
def run_replay(args, ctx):
    """Per rank (one instance each, no exchange between instances): n requests with Poisson arrivals whose prompts
    reuse a prefix of one of 10,000 pool prompts chosen by Zipf(0.9), uint32 tokens, block 64.  One step = hash every
    request, replay the whole trace in arrival order (each request hits the blocks written by earlier ones and
    writes the rest), then gather every missed block from a DeepSeek-style MLA cache (61 layers, latent 512 + rope
    64 bf16 = 1152 B per token, page = block = 64 tokens, 73,728 B per layer and block) into staging, in rounds that
    reuse one staging area."""
    import torch
    import torch.distributed as dist

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200.kernel import batch_gather_kv_pages
    from tair_kvcache_b200.manager import GenKeyVectorBatch, key_offsets, length_order
    from tair_kvcache_b200.optimizer import TRACE_DIALOG_TURN, RunTraces, replay_workspace_bytes

    rank, world, device = ctx.rank, ctx.world, ctx.device
    n_req = args.n_requests or 125000
    bs, n_prompts, n_layers, page_bytes = 64, 10000, 61, 64 * 1152
    pool_pages = args.pool_pages or 8192
    rng = np.random.default_rng(0xB2000005 + rank)
    # arrivals: exponential gaps; the trace is already in timestamp order
    prompt_len = rng.integers(256, 2049, size=n_prompts)
    req_len = rng.integers(256, 2049, size=n_req)
    zipf = 1.0 / np.arange(1, n_prompts + 1) ** 0.9
    prompt_of = rng.choice(n_prompts, size=n_req, p=zipf / zipf.sum())
    share = (rng.random(n_req) * (np.minimum(req_len, prompt_len[prompt_of]) + 1)).astype(np.int64)
    poff = np.zeros(n_prompts + 1, dtype=np.int64)
    np.cumsum(prompt_len, out=poff[1:])
    off = np.zeros(n_req + 1, dtype=np.int64)
    np.cumsum(req_len, out=off[1:])
    gen = torch.Generator(device=device).manual_seed(0xB2000005 + rank)
    prompts = torch.randint(0, 151936, (int(poff[-1]),), dtype=torch.int32, device=device, generator=gen)
    toks = torch.randint(0, 151936, (int(off[-1]),), dtype=torch.int32, device=device, generator=gen)
    # copy the shared prefixes with one indexed assignment
    d_share = torch.from_numpy(share).to(device)
    dst0 = torch.from_numpy(off[:-1]).to(device)
    src0 = torch.from_numpy(poff[prompt_of]).to(device)
    within = torch.arange(int(share.sum()), device=device) - torch.repeat_interleave(
        torch.cumsum(d_share, 0) - d_share, d_share)
    toks[torch.repeat_interleave(dst0, d_share) + within] = prompts[torch.repeat_interleave(src0, d_share) + within]
    del within, prompts

    ko = key_offsets(off, bs)
    n_keys = int(ko[-1])
    d_off, d_ko = torch.from_numpy(off).to(device), torch.from_numpy(ko).to(device)
    order_np, residency = length_order(off, with_residency=True)
    d_order = torch.from_numpy(order_np).to(device)
    d_keys = torch.empty(n_keys, dtype=torch.int64, device=device)
    d_type = torch.full((n_req,), TRACE_DIALOG_TURN, dtype=torch.uint8, device=device)
    workspace = torch.empty(replay_workspace_bytes(n_keys), dtype=torch.uint8, device=device)
    counts = torch.from_numpy(ko[1:] - ko[:-1]).to(device)
    trace_of_key = torch.repeat_interleave(torch.arange(n_req, device=device), counts)
    pos_in_trace = torch.arange(n_keys, device=device) - d_ko[:-1][trace_of_key]

    pools = [torch.empty(pool_pages * page_bytes // 4, dtype=torch.int32, device=device).random_(generator=gen)
             for _ in range(n_layers)]
    ptrs = torch.tensor([p.data_ptr() for p in pools], dtype=torch.int64, device=device)
    round_blocks = 2048  # staging area reused by every round: 2048 x 4.5 MB = 9.2 GB
    staging = torch.empty(round_blocks * n_layers * page_bytes // 4, dtype=torch.int32, device=device)

    def step():
        keys = GenKeyVectorBatch(toks, d_off, bs, d_ko, n_keys, out=d_keys, order=d_order, warps_per_sm=residency)
        res = RunTraces(keys, d_ko, d_type, workspace=workspace)
        miss = pos_in_trace >= res.external_hit_blocks[trace_of_key]
        # engine page of a missed block: derived from its key (any page serves for a bandwidth measurement)
        pages = (keys[miss] & 0x7FFFFFFF).remainder(pool_pages).to(torch.int32)
        n_miss = pages.numel()
        for a in range(0, n_miss, round_blocks):
            batch_gather_kv_pages(ptrs, staging, pages[a:a + round_blocks], None, 1, page_bytes, pool_pages)
        return res, n_miss

    for _ in range(max(1, min(args.warmup, 1))):
        res, n_miss = step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    steps = max(1, min(args.steps, 3))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        res, n_miss = step()
    e1.record()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1) / steps
    hits = int(res.external_hit_blocks.sum().item())
    stats = torch.tensor([ms, float(n_req), float(n_keys), float(hits), float(n_miss)], dtype=torch.float64,
                         device=device)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        stats[0] = mx[0]
    ms, tot_req, tot_keys, tot_hits, tot_miss = stats.tolist()

    parity = None
    if rank == 0 and not args.no_cpu:
        from oracle import kvcm_oracle as oracle
        m = min(n_req, 20000)  # the sequential CPU replay of the first requests sees the same history
        k = d_keys[:int(ko[m])].cpu().numpy()
        want = oracle.Replay().run(k, ko[:m + 1], np.zeros(m, dtype=np.uint8))
        parity = bool(np.array_equal(want[0], res.external_hit_blocks[:m].cpu().numpy()) and
                      np.array_equal(want[2], res.write_blocks[:m].cpu().numpy()))
    line = None
    if rank == 0:
        gather_bytes = 2 * tot_miss * n_layers * page_bytes
        peak, peak_kind = peaks()
        per_gpu = gather_bytes / world / (ms * 1e-3) / 1e9
        line = ({
            "metric": "mixed_replay_requests_per_s", "value": tot_req / (ms * 1e-3), "unit": "requests/s",
            "n_gpus": world, "steps": steps, "warmup": 1, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64+u8", "data": "synthetic",
            "config": {"workload": "%d requests per GPU (one instance each), 256-2048 uint32 tokens, block 64, Zipf(0.9) "
                                   "prefix reuse over 10000 prompts; hash + replay + gather of missed blocks from an MLA "
                                   "cache (61 layers x 73,728 B per block)" % n_req,
                       "token_blocks": int(tot_keys), "hit_blocks": int(tot_hits), "missed_blocks": int(tot_miss),
                       "token_blocks_per_s": tot_keys / (ms * 1e-3),
                       "instances": "%d independent instances, one per GPU, no exchange between them" % world,
                       "gather_algorithmic_GBps": gather_bytes / (ms * 1e-3) / 1e9, "parity_sample_ok": parity},
            "parity_sample_ok": parity,
            "roofline": {"bound": "hbm", "kernel": "MoveRowsBulkKernel<gather> (the step's dominant kernel: the gather "
                                                   "of the missed MLA blocks)", "achieved": per_gpu, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": per_gpu / peak, "traffic": None,
                         "note": "whole step time (hash + replay + gathers) against the gathers' algorithmic bytes"},
            "gpu_launches": int(world * (5 + (tot_miss / world + round_blocks - 1) // round_blocks))})
    return line


def window_cpu_baseline(n_requests_total, threads, budget_s=10.0):
    """The CPU side of the sliding-window configuration on a bounded sample - the same length / sharing
    distributions at 1/32 of the requests and of the index - through the reference's own searcher compiled from its
    sources where that library is there (checking its answers against the oracle's on the way), else through the
    oracle.  Returns (token-blocks/s, repetitions, cpu_baseline dict, description of what ran)."""
    from oracle import kvcm_oracle as oracle
    n_req, n_roots, bs, sw = n_requests_total // 32, 64, 16, 256
    rng = np.random.default_rng(0xB2000004)

    def loguniform(n):
        return np.exp(rng.uniform(np.log(256), np.log(131072), size=n)).astype(np.int64)

    root_len, req_len = loguniform(n_roots), loguniform(n_req)
    zipf = 1.0 / np.arange(1, n_roots + 1) ** 1.1
    root_of = rng.choice(n_roots, size=n_req, p=zipf / zipf.sum())
    roots = [rng.integers(0, 151936, size=n, dtype=np.int64).astype(np.uint32) for n in root_len]
    reqs = []
    for r in range(n_req):
        t = rng.integers(0, 151936, size=req_len[r], dtype=np.int64).astype(np.uint32)
        m = int(rng.random() * (min(req_len[r], root_len[root_of[r]]) + 1))
        t[:m] = roots[root_of[r]][:m]
        reqs.append(t)
    off = np.zeros(n_req + 1, dtype=np.int64)
    np.cumsum(req_len, out=off[1:])
    toks = np.concatenate(reqs)
    ox = oracle.Index()
    for t in roots:
        ox.put_uniform(oracle.gen_key_vector(t, bs))
    keys0, ko0 = oracle.hash_blocks(toks, off, bs, threads=threads)
    ox.put_uniform(keys0[:int(ko0[n_req // 8])])
    from oracle import ref_searcher
    t_total, n, kind = 0.0, 0, "port"
    searcher = None
    if ref_searcher.available():
        try:
            # the reference's own searcher compiled from its sources, its local meta backend in memory
            index_keys = np.unique(np.concatenate([oracle.gen_key_vector(t, bs) for t in roots] +
                                                  [keys0[:int(ko0[n_req // 8])]]))
            searcher = ref_searcher.RefSearcher(max_keys=2 * len(index_keys), in_memory=True)
            for a in range(0, len(index_keys), 20000):
                searcher.add(index_keys[a:a + 20000], 4, oracle.CLS_SERVING)
        except (OSError, RuntimeError, AttributeError) as err:  # there, but it does not load or run here
            print("reference searcher not usable (%s): timing the restatement instead" % err, file=sys.stderr)
            searcher = None
    if searcher is not None:
        kind = "reference"
        t64 = toks.astype(np.int64)
        while t_total < budget_s and n < 500:
            t0 = time.perf_counter()
            matched, base = searcher.window_match_batch(t64, off, bs, sw, threads=threads)
            t_total += time.perf_counter() - t0
            n += 1
        # the sample's answers are the oracle's (reported, not asserted: a timing run should end with its line)
        agrees = bool(np.array_equal(matched, ox.prefix_match_batch(keys0, ko0, threads=threads)) and
                      np.array_equal(base, ox.sw_match_batch(keys0, ko0, sw, threads=threads)))
    while kind == "port" and t_total < budget_s and n < 500:
        t0 = time.perf_counter()
        keys, ko = oracle.hash_blocks(toks, off, bs, threads=threads)
        ox.prefix_match_batch(keys, ko, threads=threads)
        ox.sw_match_batch(keys, ko, sw, threads=threads)
        t_total += time.perf_counter() - t0
        n += 1
    value = int(ko0[-1]) * n / t_total
    sample = "%d of %d requests (%d token blocks), index of %d keys, %d repetitions" % (
        n_req, n_requests_total, int(ko0[-1]), len(ox), n)
    what = ("the reference's own GenKeyVector + MetaSearcher::PrefixMatch + ReverseRollSlideWindowMatch compiled from "
            "its sources (local meta backend in memory)" if kind == "reference" else
            "CPU restatement (hash + prefix + sliding-window match, without the reference's per-key JSON parse)")
    base = {"value": value, "unit": "token-blocks/s", "cores": threads, "kind": kind, "sample": sample + "; " + what}
    if kind == "reference":
        base["reference_equals_oracle"] = agrees
    return value, n, base, what


def main_window_reference(args):
    """CPU arm of --workload c4."""
    threads = os.cpu_count() or 1
    value, n, base, what = window_cpu_baseline(args.n_requests or 65536, threads)
    print(json.dumps({"impl": "reference", "metric": "prefix_and_window_match_token_blocks_per_s", "value": value,
                      "unit": "token-blocks/s", "n_gpus": args.gpus, "steps": n, "warmup": 0, "higher_is_better": True,
                      "dtype": "int64", "data": "synthetic",
                      "config": {"workload": what + " on a bounded sample"},
                      "cpu_baseline": base,
                      "e2e": {"value": value, "unit": "token-blocks/s", "h2d_bytes_per_step": 0,
                              "d2h_bytes_per_step": 0}, "gpu_launches": 0}))


def main_replay_reference(args):
    """CPU arm of --workload c5 on a bounded sample: hash, sequential prefix-tree replay (one core, as the reference
    replays), and a memcpy gather of the missed blocks from host-resident MLA pools with all host threads."""
    from oracle import kvcm_oracle as oracle
    threads = os.cpu_count() or 1
    n_req, bs, n_prompts, n_layers, page_bytes, pool_pages = 2000, 64, 500, 61, 64 * 1152, 256
    rng = np.random.default_rng(0xB2000005)
    prompt_len = rng.integers(256, 2049, size=n_prompts)
    req_len = rng.integers(256, 2049, size=n_req)
    zipf = 1.0 / np.arange(1, n_prompts + 1) ** 0.9
    prompt_of = rng.choice(n_prompts, size=n_req, p=zipf / zipf.sum())
    prompts = [rng.integers(0, 151936, size=n, dtype=np.int64).astype(np.uint32) for n in prompt_len]
    reqs = []
    for r in range(n_req):
        t = rng.integers(0, 151936, size=req_len[r], dtype=np.int64).astype(np.uint32)
        m = int(rng.random() * (min(req_len[r], prompt_len[prompt_of[r]]) + 1))
        t[:m] = prompts[prompt_of[r]][:m]
        reqs.append(t)
    off = np.zeros(n_req + 1, dtype=np.int64)
    np.cumsum(req_len, out=off[1:])
    toks = np.concatenate(reqs)
    pools = [rng.integers(0, 256, size=pool_pages * page_bytes, dtype=np.uint8) for _ in range(n_layers)]
    staging = np.zeros(128 * n_layers * page_bytes, dtype=np.uint8)
    t_total, n, n_miss = 0.0, 0, 0
    while t_total < 10.0 and n < 10:
        t0 = time.perf_counter()
        keys, ko = oracle.hash_blocks(toks, off, bs, threads=threads)
        ext, _, wr, _ = oracle.Replay().run(keys, ko, np.zeros(n_req, dtype=np.uint8))
        miss = np.concatenate([keys[ko[r] + ext[r]:ko[r + 1]] for r in range(n_req)])
        pages = ((miss & 0x7FFFFFFF) % pool_pages).astype(np.int32)
        for a in range(0, len(pages), 128):
            chunk = pages[a:a + 128]
            oracle.move_rows(pools, staging, chunk, None, 1, page_bytes, 0, threads=threads)
        t_total += time.perf_counter() - t0
        n, n_miss = n + 1, len(pages)
    value = n_req * n / t_total
    print(json.dumps({"impl": "reference", "metric": "mixed_replay_requests_per_s", "value": value, "unit": "requests/s",
                      "n_gpus": args.gpus, "steps": n, "warmup": 0, "higher_is_better": True, "dtype": "int64+u8",
                      "data": "synthetic",
                      "config": {"workload": "CPU restatement (hash + sequential replay + memcpy gather of misses from "
                                             "host-resident MLA pools) on a bounded sample"},
                      "cpu_baseline": {"value": value, "unit": "requests/s", "cores": threads, "kind": "port",
                                       "sample": "%d requests, %d missed blocks of 4.5 MB per step, %d repetitions"
                                                 % (n_req, n_miss, n)},
                      "e2e": {"value": value, "unit": "requests/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


def _lru_trace(n_req, seed, n_prompts=10000, bs=64):
    """Token lengths and prefix sharing of the mixed-replay workload (Zipf(0.9) reuse over a prompt pool), as numpy
    arrays: request offsets, prompt offsets, the prompt each request shares a prefix with and how many tokens."""
    rng = np.random.default_rng(seed)
    prompt_len = rng.integers(256, 2049, size=n_prompts)
    req_len = rng.integers(256, 2049, size=n_req)
    zipf = 1.0 / np.arange(1, n_prompts + 1) ** 0.9
    prompt_of = rng.choice(n_prompts, size=n_req, p=zipf / zipf.sum())
    share = (rng.random(n_req) * (np.minimum(req_len, prompt_len[prompt_of]) + 1)).astype(np.int64)
    poff = np.zeros(n_prompts + 1, dtype=np.int64)
    np.cumsum(prompt_len, out=poff[1:])
    off = np.zeros(n_req + 1, dtype=np.int64)
    np.cumsum(req_len, out=off[1:])
    return off, poff, prompt_of, share


def _lru_quotas(n_keys, n_configs):
    """Quota points of a tradeoff curve: evenly spaced fractions of the blocks the trace writes in total."""
    return [max(100, int(n_keys * (c + 1) / (2 * n_configs))) for c in range(n_configs)]


def main_lru(args, ctx):
    """Tradeoff-curve sweep of the Optimizer: the mixed-replay trace (dialog turns, block 64) replayed with the "lru"
    policy once per quota point, all points of this rank in one launch (one warp each).  Ranks take different
    quota points of the same curve (no exchange).  One step = hash the trace + the whole sweep."""
    import torch
    import torch.distributed as dist

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200.manager import GenKeyVectorBatch, key_offsets, length_order
    from tair_kvcache_b200.optimizer import (TRACE_DIALOG_TURN, RunTracesLru, RunTracesLruGroup,
                                             replay_lru_workspace_bytes)

    rank, world, device, local = ctx.rank, ctx.world, ctx.device, ctx.local
    n_req = args.n_requests or 125000
    n_cfg = args.n_configs or 148
    bs = 64
    off, poff, prompt_of, share = _lru_trace(n_req, 0xB2000005)
    gen = torch.Generator(device=device).manual_seed(0xB2000005)
    prompts = torch.randint(0, 151936, (int(poff[-1]),), dtype=torch.int32, device=device, generator=gen)
    toks = torch.randint(0, 151936, (int(off[-1]),), dtype=torch.int32, device=device, generator=gen)
    d_share = torch.from_numpy(share).to(device)
    within = torch.arange(int(share.sum()), device=device) - torch.repeat_interleave(
        torch.cumsum(d_share, 0) - d_share, d_share)
    toks[torch.repeat_interleave(torch.from_numpy(off[:-1]).to(device), d_share) + within] = prompts[
        torch.repeat_interleave(torch.from_numpy(poff[prompt_of]).to(device), d_share) + within]
    del within, prompts
    ko = key_offsets(off, bs)
    n_keys = int(ko[-1])
    d_off, d_ko = torch.from_numpy(off).to(device), torch.from_numpy(ko).to(device)
    order_np, residency = length_order(off, with_residency=True)
    d_order = torch.from_numpy(order_np).to(device)
    d_keys = torch.empty(n_keys, dtype=torch.int64, device=device)
    d_type = torch.full((n_req,), TRACE_DIALOG_TURN, dtype=torch.uint8, device=device)
    all_quotas = _lru_quotas(n_keys, n_cfg * world)
    quotas = all_quotas[rank::world]  # every rank gets points from the whole range
    policy = args.policy
    n_inst = max(1, args.instances)  # > 1: the requests go round-robin to instances that share the quota
    d_inst = (torch.arange(n_req, device=device, dtype=torch.int32) % n_inst).contiguous()
    ws_bytes = replay_lru_workspace_bytes(n_keys, n_cfg, policy, n_req)
    if n_inst > 1 and policy == "leaf_aware_lru":
        from tair_kvcache_b200 import _cabi
        ws_bytes = _cabi.lib().kvcm_b200_replay_leaf_lru_group_workspace_bytes(n_keys, n_req, n_cfg, n_inst)
    if n_inst > 1 and policy == "random_lru":
        from tair_kvcache_b200 import _cabi
        ws_bytes = _cabi.lib().kvcm_b200_replay_random_lru_group_workspace_bytes(n_keys, n_cfg, n_inst)
    workspace = torch.empty(ws_bytes + 4096, dtype=torch.uint8, device=device)
    status = torch.zeros(4, dtype=torch.int32, device=device)

    def sweep(keys):
        if n_inst > 1:
            return RunTracesLruGroup(keys, d_ko, d_type, d_inst, n_inst, quotas, evict_batch=100, mode=1,
                                     workspace=workspace, status=status, policy=policy)
        return RunTracesLru(keys, d_ko, d_type, quotas, evict_batch=100, precise=False, workspace=workspace,
                            status=status, policy=policy)

    def step():
        keys = GenKeyVectorBatch(toks, d_off, bs, d_ko, n_keys, out=d_keys, order=d_order, warps_per_sm=residency)
        return sweep(keys)

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(max(1, min(args.warmup, 3))):
        res = step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    steps = max(1, min(args.steps, 5))
    if sampler:
        sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        res = step()
    e1.record()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_end()
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1) / steps
    # the sweep kernel alone
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    sweep(d_keys)
    e3.record()
    torch.cuda.synchronize(device)
    sweep_ms = e2.elapsed_time(e3)
    hit_rate = (res.totals[:, 0].double() / max(n_keys, 1)).cpu().numpy()
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    parity = None
    if rank == 0 and not args.no_cpu:
        from oracle import kvcm_oracle as oracle
        m = min(n_req, 20000)  # the sequential CPU replay of the first requests sees the same history
        k = d_keys[:int(ko[m])].cpu().numpy()
        c = len(quotas) // 3
        if n_inst > 1:
            want = oracle.LruGroupReplay(quotas[c], n_inst, evict_batch=100, mode=1, policy=policy).run(
                k, ko[:m + 1], np.zeros(m, np.uint8), np.arange(m, dtype=np.int32) % n_inst)
        else:
            want = oracle.LruReplay(quotas[c], evict_batch=100, precise=False, policy=policy).run(
                k, ko[:m + 1], np.zeros(m, np.uint8))
        parity = bool(np.array_equal(want[0], res.external_hit_blocks[c, :m].cpu().numpy()) and
                      np.array_equal(want[2], res.write_blocks[c, :m].cpu().numpy()) and
                      np.array_equal(want[3], res.current_cache_blocks[c, :m].cpu().numpy()))
    if rank == 0:
        replays = n_req * n_cfg * world
        print(json.dumps({
            "metric": "%s_tradeoff_sweep_request_replays_per_s" % policy, "value": replays / (ms / 1e3),
            "unit": "request-replays/s", "n_gpus": world, "steps": steps, "warmup": max(1, min(args.warmup, 3)),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int64", "data": "synthetic",
            "config": {"workload": "%d requests (dialog turns, 256-2048 uint32 tokens, block 64, Zipf(0.9) prefix "
                                   "reuse over 10000 prompts = %d token blocks) replayed with %s eviction at %d quota "
                                   "points per GPU (%d..%d blocks, rough mode, batches of 100); hash + sweep per step"
                                   % (n_req, n_keys, policy, n_cfg, min(all_quotas), max(all_quotas)),
                       "instances_sharing_the_quota": n_inst,
                       "sweep_kernel_ms_rank0": sweep_ms, "hit_rate_lowest_quota": float(hit_rate[0]),
                       "hit_rate_highest_quota": float(hit_rate[-1]), "table_overflows": int(status[0].item()),
                       "parity_sample_ok": parity},
            # per step: the hash, then table init + claim + lookup + sweep ("lru"), one more pass for the key
            # positions ("leaf_aware_lru"), or extents / instance check + (clear, claim, lookup) per instance + sweep
            # (groups; one more pass for the key positions under "leaf_aware_lru")
            "clocks": clocks,
            "gpu_launches": ((3 * n_inst + (4 if policy == "leaf_aware_lru" else 3)) if n_inst > 1
                             else 6 if policy == "leaf_aware_lru" else 5) * steps}))


def main_lru_reference(args):
    """CPU arm of --workload lru on a bounded sample: the first requests of the same trace hashed and replayed with
    the radix tree + LRU restatement, one quota point per host thread at a time (the reference's tradeoff scripts
    likewise run one optimizer per point in a thread pool)."""
    from concurrent.futures import ThreadPoolExecutor

    from oracle import kvcm_oracle as oracle
    threads = os.cpu_count() or 1
    n_req_full = args.n_requests or 125000
    n_req, bs = min(n_req_full, 20000), 64
    n_cfg = min(args.n_configs or 148, 2 * threads)
    off, poff, prompt_of, share = _lru_trace(n_req_full, 0xB2000005)
    off = off[:n_req + 1]
    rng = np.random.default_rng(0xB2000005)
    prompts = rng.integers(0, 151936, size=int(poff[-1]), dtype=np.int64).astype(np.uint32)
    toks = rng.integers(0, 151936, size=int(off[-1]), dtype=np.int64).astype(np.uint32)
    for r in range(n_req):
        toks[off[r]:off[r] + share[r]] = prompts[poff[prompt_of[r]]:poff[prompt_of[r]] + share[r]]
    types = np.zeros(n_req, dtype=np.uint8)
    t0 = time.perf_counter()
    keys, ko = oracle.hash_blocks(toks, off, bs, threads=threads)
    quotas = _lru_quotas(int(ko[-1]), n_cfg)

    from oracle import ref_optimizer
    compiled = ref_optimizer.available()  # the reference's own Optimizer, compiled from its sources (oracle/_ref)
    n_inst = max(1, args.instances)
    inst = np.arange(n_req, dtype=np.int32) % n_inst

    def one(q):
        if compiled:
            r = ref_optimizer.RefOptimizer([dict(quota_capacity=q, instances=[(str(j), args.policy)
                                                                              for j in range(n_inst)])],
                                           evict_batch=100, mode=1 if n_inst > 1 else 2)
            return int(r.run(keys, ko, types, inst)[0].sum())
        if n_inst > 1:
            return int(oracle.LruGroupReplay(q, n_inst, evict_batch=100, mode=1, policy=args.policy).run(
                keys, ko, types, inst)[0].sum())
        return int(oracle.LruReplay(q, evict_batch=100, precise=False, policy=args.policy).run(keys, ko, types)[0].sum())

    with ThreadPoolExecutor(max_workers=threads) as pool:
        hits = list(pool.map(one, quotas))
    dt = time.perf_counter() - t0
    value = n_req * n_cfg / dt
    sample = "first %d of %d requests (%d token blocks), %d quota points, hit blocks %d..%d" % (
        n_req, n_req_full, int(ko[-1]), n_cfg, min(hits), max(hits))
    print(json.dumps({"impl": "reference", "metric": "%s_tradeoff_sweep_request_replays_per_s" % args.policy,
                      "value": value,
                      "unit": "request-replays/s", "n_gpus": args.gpus, "steps": 1, "warmup": 0,
                      "higher_is_better": True, "dtype": "int64", "data": "synthetic",
                      "config": {"workload": "%s (hash + radix tree with %s eviction, one quota point per thread) on "
                                             "a bounded sample" % ("the reference's Optimizer compiled from its own "
                                                                   "sources" if compiled else "CPU restatement",
                                                                   args.policy)},
                      "cpu_baseline": {"value": value, "unit": "request-replays/s", "cores": threads,
                                       "kind": "reference" if compiled else "port", "sample": sample},
                      "e2e": {"value": value, "unit": "request-replays/s", "h2d_bytes_per_step": 0,
                              "d2h_bytes_per_step": 0}, "gpu_launches": 0}))


def main_iov(args, ctx):
    """TransferClient side (the per-iov copy loops of LocalFileSdk::DoGet / DoPut and Hf3fsUsrbioClient::CopyIovs):
    blocks of layer_num x (K, V) iovs <-> contiguous block strings, at the Llama-3-8B shape (64 iovs of 128 KiB per
    block, 2,048 blocks = 131,072 iovs, 16 GiB).  One step = Put (iovs -> strings) + Get (strings -> iovs), each one
    kvcm_b200_copy_segments launch.  Beside it, on the same buffers: the reference's own structure, one
    cudaMemcpyAsync per iov, on a bounded number of blocks."""
    import ctypes

    import torch
    import torch.distributed as dist

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200 import _cabi

    rank, world, device, local = ctx.rank, ctx.world, ctx.device, ctx.local
    _cabi.bind_device(local)
    n_blocks = args.n_blocks or 2048
    n_iovs, iov_bytes = 64, 64 * 2048  # 32 layers x (K, V); 64 tokens x 2 KiB
    block_bytes = n_iovs * iov_bytes
    gen = torch.Generator(device=device).manual_seed(0xB2000002 + rank)
    # engine side: one buffer per (layer, K/V) holding that iov of every block, blocks at permuted positions
    bufs = [torch.empty(n_blocks * iov_bytes // 4, dtype=torch.int32, device=device).random_(generator=gen)
            for _ in range(n_iovs)]
    strings = torch.zeros(n_blocks * block_bytes // 4, dtype=torch.int32, device=device)
    perm = np.random.default_rng(0xB2000002 + rank).permutation(n_blocks)
    base = np.array([b.data_ptr() for b in bufs], dtype=np.uint64)
    iov_addr = base[None, :] + (perm.astype(np.uint64) * np.uint64(iov_bytes))[:, None]          # [block, iov]
    str_addr = np.uint64(strings.data_ptr()) + (np.arange(n_blocks, dtype=np.uint64) * np.uint64(block_bytes))[:, None] \
        + (np.arange(n_iovs, dtype=np.uint64) * np.uint64(iov_bytes))[None, :]

    def seg_table(dst, src):
        t = np.empty((n_blocks * n_iovs, 3), dtype=np.uint64)
        t[:, 0], t[:, 1], t[:, 2] = dst.reshape(-1), src.reshape(-1), iov_bytes
        return torch.from_numpy(t.view(np.uint8).reshape(-1)).to(device)

    put_segs, get_segs = seg_table(str_addr, iov_addr), seg_table(iov_addr, str_addr)
    n_segs = n_blocks * n_iovs
    stream = torch.cuda.current_stream(device).cuda_stream

    def put():
        _cabi.call("kvcm_b200_copy_segments_sized", put_segs.data_ptr(), n_segs, n_segs * iov_bytes, stream)

    def get():
        _cabi.call("kvcm_b200_copy_segments_sized", get_segs.data_ptr(), n_segs, n_segs * iov_bytes, stream)

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
    put()
    torch.cuda.synchronize(device)
    # parity: a sample of block strings against a torch gather of the iov buffers
    ok = True
    for b in np.random.default_rng(1).choice(n_blocks, size=min(16, n_blocks), replace=False):
        want = torch.stack([buf.view(n_blocks, -1)[int(perm[b])] for buf in bufs]).reshape(-1)
        ok = ok and bool(torch.equal(strings.view(n_blocks, -1)[int(b)], want))
    for _ in range(args.warmup):
        put()
        get()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_begin()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    for k in range(args.steps):
        ev[k][0].record()
        put()
        ev[k][1].record()
        get()
        ev[k][2].record()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_end()
    clocks = sampler.stop() if sampler else None
    put_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    get_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    if world > 1:
        t = torch.tensor([total_ms, put_ms, get_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, put_ms, get_ms = t.tolist()
    payload = n_blocks * block_bytes
    value = world * 4 * payload * args.steps / (total_ms * 1e-3) / 1e9

    # the reference's structure on the same buffers: one cudaMemcpyAsync per iov, then one stream sync
    # (a compiled loop under oracle/, so that no interpreter overhead is charged to it)
    loop_gbs = loop_calls = loop_us = None
    loop_lib = os.path.join(ROOT, "oracle", "libkvcm_ref_memcpy_loop.so")
    if rank == 0 and os.path.exists(loop_lib):
        rt = ctypes.CDLL(loop_lib)
        rt.kvcm_ref_memcpy_loop.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_void_p]
        m = min(n_blocks, 512)
        dsts = np.ascontiguousarray(str_addr[:m].reshape(-1))
        srcs = np.ascontiguousarray(iov_addr[:m].reshape(-1))
        sizes = np.full(len(dsts), iov_bytes, dtype=np.uint64)
        torch.cuda.synchronize(device)
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            rc = rt.kvcm_ref_memcpy_loop(dsts.ctypes.data, srcs.ctypes.data, sizes.ctypes.data, len(dsts), stream)
            dt = time.perf_counter() - t0
            best = dt if best is None or dt < best else best
        loop_calls = len(dsts)
        if rc == 0:
            loop_gbs, loop_us = 2 * m * block_bytes / best / 1e9, best / loop_calls * 1e6

    # end to end: block strings in pinned host memory (LocalFileSdk registers its mmap'ed file with the driver).
    # As the IovCopier adapter does: the strings cross PCIe as one copy-engine transfer into / out of a device
    # bounce buffer and the kernel runs device to device; Put on one stream, Get on another.
    e2e = None
    if not args.no_e2e:
        m = min(n_blocks, 128)
        words = m * block_bytes // 4
        h_str = torch.empty(words, dtype=torch.int32, pin_memory=True)
        h_back = strings[:words].cpu().pin_memory()
        d_put_b, d_get_b = torch.empty(words, dtype=torch.int32, device=device), torch.empty(
            words, dtype=torch.int32, device=device)
        rel = str_addr[:m] - np.uint64(strings.data_ptr())

        def small(dst, src):
            t = np.empty((m * n_iovs, 3), dtype=np.uint64)
            t[:, 0], t[:, 1], t[:, 2] = dst.reshape(-1), src.reshape(-1), iov_bytes
            return torch.from_numpy(t.view(np.uint8).reshape(-1)).pin_memory()

        h_put = small(np.uint64(d_put_b.data_ptr()) + rel, iov_addr[:m])
        h_get = small(iov_addr[:m], np.uint64(d_get_b.data_ptr()) + rel)
        d_put, d_get = torch.empty_like(h_put, device=device), torch.empty_like(h_get, device=device)
        s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

        def e2e_step():
            with torch.cuda.stream(s1):
                d_put.copy_(h_put, non_blocking=True)  # the segment table crosses PCIe with every request
                _cabi.call("kvcm_b200_copy_segments_sized", d_put.data_ptr(), m * n_iovs, m * block_bytes, s1.cuda_stream)
                h_str.copy_(d_put_b, non_blocking=True)
            with torch.cuda.stream(s2):
                d_get.copy_(h_get, non_blocking=True)
                d_get_b.copy_(h_back, non_blocking=True)
                _cabi.call("kvcm_b200_copy_segments_sized", d_get.data_ptr(), m * n_iovs, m * block_bytes, s2.cuda_stream)

        e2e_step()
        torch.cuda.synchronize(device)
        reps = max(1, min(args.steps, 3))
        ctx.barrier()  # every rank crosses the host link during the same interval; the slowest one counts
        t0 = time.perf_counter()
        for _ in range(reps):
            e2e_step()
        torch.cuda.synchronize(device)
        dt = ctx.max_over_ranks([time.perf_counter() - t0])[0]
        e2e = {"value": world * 4 * m * block_bytes * reps / dt / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": m * block_bytes + 2 * m * n_iovs * 24, "d2h_bytes_per_step": m * block_bytes,
               "parity_ok": bool(torch.equal(h_str, h_back))}
    if rank != 0:
        return
    peak, peak_kind = peaks()
    kern = 2 * payload / (min(put_ms, get_ms) * 1e-3) / 1e9
    line = {"metric": "iov_copy_algorithmic_GBps", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "%d blocks x %d iovs x %d KiB (Llama-3-8B block layout), Put + Get per step, block "
                                   "strings and iov buffers in HBM, inputs larger than L2" % (n_blocks, n_iovs,
                                                                                             iov_bytes // 1024),
                       "put_ms": put_ms, "get_ms": get_ms, "parity_sample_ok": ok,
                       "memcpy_async_per_iov_GBps": loop_gbs, "memcpy_async_calls": loop_calls,
                       "memcpy_async_us_per_call": loop_us},
            "roofline": {"bound": "hbm", "kernel": "CopySegmentsBulkKernel", "achieved": kern, "peak": peak, "unit": UNIT,
                         "frac": kern / peak, "traffic": int(2 * payload * IOV_DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE),
                         "traffic_source": "ncu capture on 256 blocks scaled by blocks moved",
                         "algorithmic_bytes_per_launch": 2 * payload, "peak_kind": peak_kind},
            "clocks": clocks, "gpu_launches": 2 * args.steps}
    if e2e:
        line["e2e"] = e2e
    print(json.dumps(line))


def main_iov_reference(args):
    """CPU arm of --workload iov: the same per-iov loop with memcpy between host buffers (oracle.copy_iovs), on a
    bounded number of blocks, all host threads (one block per task)."""
    from concurrent.futures import ThreadPoolExecutor

    from oracle import kvcm_oracle as oracle
    threads = os.cpu_count() or 1
    n_iovs, iov_bytes, m = 64, 64 * 2048, 64
    rng = np.random.default_rng(0xB2000002)
    bufs = [[rng.integers(0, 256, size=iov_bytes, dtype=np.uint8) for _ in range(n_iovs)] for _ in range(m)]
    strings = [np.zeros(n_iovs * iov_bytes, dtype=np.uint8) for _ in range(m)]

    def one(b):
        oracle.copy_iovs([(v, iov_bytes, False) for v in bufs[b]], strings[b], 0)
        oracle.copy_iovs([(v, iov_bytes, False) for v in bufs[b]], strings[b], 1)

    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(one, range(m)))
        t_total, n = 0.0, 0
        while t_total < 5.0 and n < 50:
            t0 = time.perf_counter()
            list(pool.map(one, range(m)))
            t_total += time.perf_counter() - t0
            n += 1
    value = 4 * m * n_iovs * iov_bytes * n / t_total / 1e9
    print(json.dumps({"impl": "reference", "metric": "iov_copy_algorithmic_GBps", "value": value, "unit": UNIT,
                      "n_gpus": args.gpus, "steps": n, "warmup": 1, "higher_is_better": True, "dtype": "u8",
                      "data": "synthetic",
                      "config": {"workload": "CPU restatement of the per-iov loop (memcpy between host buffers)"},
                      "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                                       "sample": "%d blocks x %d iovs x %d KiB, Put + Get, %d repetitions" % (
                                           m, n_iovs, iov_bytes // 1024, n)},
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


def main_hash(args, ctx):
    """Chained block hash alone on a batch with many more requests than schedulers (the regime where the integer pipe,
    not one request's dependent chain, sets the pace): n requests of the same length, uint32 tokens, block 16.
    Ranks hash different requests (no exchange)."""
    import torch
    import torch.distributed as dist

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200.manager import GenKeyVectorBatch, key_offsets

    rank, world, device, local = ctx.rank, ctx.world, ctx.device, ctx.local
    n_req, length, bs = args.n_requests or 65536, args.request_tokens or 20970, 16
    off = np.arange(n_req + 1, dtype=np.int64) * length
    gen = torch.Generator(device=device).manual_seed(0xB2000006 + rank)
    toks = torch.randint(0, 151936, (n_req * length,), dtype=torch.int32, device=device, generator=gen)
    ko = key_offsets(off, bs)
    n_keys = int(ko[-1])
    d_off, d_ko = torch.from_numpy(off).to(device), torch.from_numpy(ko).to(device)
    d_keys = torch.empty(n_keys, dtype=torch.int64, device=device)

    def step():
        GenKeyVectorBatch(toks, d_off, bs, d_ko, n_keys, out=d_keys)

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(args.warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.mark_end()
    clocks = sampler.stop() if sampler else None
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    parity = None
    if rank == 0 and not args.no_cpu:
        from oracle import kvcm_oracle as oracle
        m = min(n_req, 64)
        want, _ = oracle.hash_blocks(toks[:m * length].cpu().numpy().view(np.uint32), off[:m + 1], bs, threads=4)
        parity = bool(np.array_equal(want, d_keys[:int(ko[m])].cpu().numpy()))
    if rank == 0:
        peak, peak_kind = peaks()
        achieved = (n_req * length * 4 + n_keys * 8) / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "chained_block_hash_tokens_per_s", "value": world * n_req * length / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": {"workload": "%d requests x %d uint32 tokens per GPU, block %d, %d keys; hash only, tokens "
                                   "(%.1f GB) far larger than L2" % (n_req, length, bs, n_keys,
                                                                      n_req * length * 4 / 1e9),
                       "parity_sample_ok": parity},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind,
                         "note": "the binding resource is the integer pipe (~14 instructions per token)"},
            "clocks": clocks, "gpu_launches": args.steps}))


def main_hash_reference(args):
    """CPU arm of --workload hash: the same chain on a bounded sample of the requests, all host threads."""
    from oracle import kvcm_oracle as oracle
    threads = os.cpu_count() or 1
    n_req_full, length, bs = args.n_requests or 65536, args.request_tokens or 20970, 16
    n_req = min(n_req_full, 2048)
    off = np.arange(n_req + 1, dtype=np.int64) * length
    toks = np.random.default_rng(0xB2000006).integers(0, 151936, size=n_req * length, dtype=np.int64).astype(np.uint32)
    oracle.hash_blocks(toks, off, bs, threads=threads)
    t_total, n = 0.0, 0
    while t_total < 10.0 and n < 200:
        t0 = time.perf_counter()
        oracle.hash_blocks(toks, off, bs, threads=threads)
        t_total += time.perf_counter() - t0
        n += 1
    value = n_req * length * n / t_total
    print(json.dumps({"impl": "reference", "metric": "chained_block_hash_tokens_per_s", "value": value,
                      "unit": "tokens/s", "n_gpus": args.gpus, "steps": n, "warmup": 1, "higher_is_better": True,
                      "dtype": "int64", "data": "synthetic",
                      "config": {"workload": "CPU restatement of GenKeyVector, one request per task"},
                      "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                                       "sample": "%d of %d requests x %d tokens, %d repetitions" % (
                                           n_req, n_req_full, length, n)},
                      "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


def _route_workload(n_ranks, keys_per_rank, seed=0xB2000007):
    """Per emulated rank: requests of 64-512 keys whose keys are stored with probability 0.8 in runs (so that
    prefixes and windows exist), as int64 arrays.  Returns (stored keys, [(keys, key_off)] per rank)."""
    rng = np.random.default_rng(seed)
    stored, batches = [], []
    for _ in range(n_ranks):
        lens = rng.integers(64, 513, size=keys_per_rank // 288 + 1)
        off = np.zeros(len(lens) + 1, dtype=np.int64)
        np.cumsum(lens, out=off[1:])
        keys = rng.integers(-(1 << 62), 1 << 62, size=int(off[-1]), dtype=np.int64)
        run = np.repeat(rng.random(len(keys) // 16 + 1) < 0.8, 16)[:len(keys)]  # hits and misses in runs of 16
        stored.append(keys[run])
        batches.append((keys, off))
    return np.concatenate(stored), batches


def main_route(args, rank):
    """The routed exchange's kernels on ONE GPU: R ranks' shards and exchange areas live in one process, attached
    to each other, and a step runs what the R ranks of a box run between their meeting points - count and dispatch
    of every rank, answer of every rank, collect and both matchers of every rank.  Peer stores land in this GPU's
    own memory, so the figures are the kernels' HBM-side cost; the NVLink share is measured by --workload c4."""
    import ctypes

    import torch

    import tair_kvcache_b200  # noqa: F401
    from tair_kvcache_b200 import _cabi
    from tair_kvcache_b200.manager import CudaShardBackend, encode_locations

    if rank != 0:
        return
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    R, per_rank, sw = 8, args.n_requests or 8_000_000, 16
    stored, batches = _route_workload(R, per_rank)
    word = encode_locations([(3, 4)])
    shards = [CudaShardBackend(len(stored) // R * 2 + 1024, device) for _ in range(R)]
    d_stored = torch.from_numpy(stored).to(device)
    for r, sh in enumerate(shards):
        sh.upsert_owned(d_stored, word, R, r)
    del d_stored
    d_keys = [torch.from_numpy(k).to(device) for k, _ in batches]
    d_off = [torch.from_numpy(o).to(device) for _, o in batches]
    n_keys = sum(len(k) for k, _ in batches)
    cap = int(max(len(k) for k, _ in batches) * 1.25) + 65536
    areas = [sh.route_area_create(cap) for sh in shards]
    handles = (ctypes.c_void_p * R)(*[a.value for a in areas])
    for r, a in enumerate(areas):
        _cabi.call("kvcm_b200_route_area_attach_local", a, R, r, handles)
    matrix = np.stack([sh.route_count(k, R).cpu().numpy() for sh, k in zip(shards, d_keys)]).astype(np.uint32)
    phase = {"count": 0.0, "dispatch": 0.0, "answer": 0.0, "collect": 0.0, "match_from_flags": 0.0}
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    out = {}

    def step(timed=False):
        ev[0].record()
        for sh, k in zip(shards, d_keys):
            sh.route_count(k, R)
        ev[1].record()
        pos = [sh.route_dispatch(a, k, matrix) for sh, a, k in zip(shards, areas, d_keys)]
        ev[2].record()
        for sh, a in zip(shards, areas):
            sh.route_answer(a, matrix)
        ev[3].record()
        flags = [sh.route_collect(a, p) for sh, a, p in zip(shards, areas, pos)]
        ev[4].record()
        out["prefix"] = [sh.prefix_from_flags(f, o, None) for sh, f, o in zip(shards, flags, d_off)]
        out["window"] = [sh.sw_from_flags(f, o, sw) for sh, f, o in zip(shards, flags, d_off)]
        out["flags"] = flags
        ev[5].record()
        if timed:
            torch.cuda.synchronize(device)
            for i, k in enumerate(phase):
                phase[k] += ev[i].elapsed_time(ev[i + 1])

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid))
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(device)
    sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(device)
    sampler.mark_end()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    for _ in range(3):
        step(timed=True)
    phase = {k: v / 3 for k, v in phase.items()}
    prefix0, window0, flags0 = (out["prefix"][0].cpu().numpy(), out["window"][0].cpu().numpy(),
                                out["flags"][0].cpu().numpy())

    # ---- end to end: every rank's keys start in pinned host memory, its match results end there
    e2e = None
    if not args.no_e2e:
        h_keys = [torch.from_numpy(k).pin_memory() for k, _ in batches]
        h_out = [torch.empty(2 * (len(o) - 1), dtype=torch.int32).pin_memory() for _, o in batches]

        def e2e_step():
            for d, h in zip(d_keys, h_keys):
                d.copy_(h, non_blocking=True)
            step()
            for r, h in enumerate(h_out):
                n_req = h.numel() // 2
                h[:n_req].copy_(out["prefix"][r], non_blocking=True)
                h[n_req:].copy_(out["window"][r], non_blocking=True)

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize(device)
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize(device)
        e2e_ms = e0.elapsed_time(e1) / args.steps
        e2e = {"value": n_keys / (e2e_ms * 1e-3), "unit": "token-blocks/s", "h2d_bytes_per_step": n_keys * 8,
               "d2h_bytes_per_step": int(sum(h.numel() for h in h_out)) * 4,
               "parity_ok": bool(np.array_equal(h_out[0][:len(prefix0)].numpy(), prefix0))}

    # ---- parity and CPU side on a sample: the first requests of rank 0 against the unsharded oracle index
    parity, cpu = None, None
    if not args.no_cpu:
        from oracle import kvcm_oracle as oracle
        threads = os.cpu_count() or 1
        keys0, off0 = batches[0]
        m = min(len(off0) - 1, 4096)
        sk, so = keys0[:int(off0[m])], off0[:m + 1]
        ox = oracle.Index()
        ox.put_uniform(sk[np.isin(sk, stored)])  # random 62-bit keys: the sample's keys decide its answers
        parity = bool(np.array_equal(ox.batch_get(sk), flags0[:len(sk)]) and
                      np.array_equal(ox.prefix_match_batch(sk, so), prefix0[:m]) and
                      np.array_equal(ox.sw_match_batch(sk, so, sw), window0[:m]))
        t_total, n = 0.0, 0
        while t_total < 5.0 and n < 2000:
            t0 = time.perf_counter()
            ox.prefix_match_batch(sk, so, threads=threads)
            ox.sw_match_batch(sk, so, sw, threads=threads)
            t_total += time.perf_counter() - t0
            n += 1
        cpu = {"value": len(sk) * n / t_total, "unit": "token-blocks/s", "cores": threads, "kind": "port",
               "sample": "prefix + window match of %d requests (%d keys) of rank 0 on an index holding their stored "
                         "keys (much smaller than the sharded one, so this over-states the CPU), %d repetitions"
                         % (m, len(sk), n)}
    peak, peak_kind = peaks()
    achieved = n_keys * 20 / (phase["dispatch"] * 1e-3) / 1e9
    print(json.dumps({
        "metric": "routed_prefix_and_window_match_token_blocks_per_s", "value": n_keys / (ms * 1e-3),
        "unit": "token-blocks/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": {"workload": "%d ranks' shards and exchange areas on one GPU; per rank %d requests of 64-512 keys "
                               "(%d keys in all, 80 %% stored, %d keys per shard); count + dispatch + answer + collect "
                               "+ prefix and window (%d) match over the flag bytes; keys (%.2f GB) and shards larger "
                               "than L2" % (R, len(batches[0][1]) - 1, n_keys, len(stored) // R, sw, n_keys * 8 / 1e9),
                   "phase_ms": phase, "parity_sample_ok": parity},
        "roofline": {"bound": "hbm", "kernel": "RouteDispatchKernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": n_keys // R * 20, "launch_ms": phase["dispatch"] / R,
                     "note": "20 B per key: key read, key stored into the owner's inbox, answer position written; the "
                             "step's longest phase is the answer kernel, bound by random probes"},
        "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": 6 * R * args.steps}))
    torch.cuda.synchronize(device)
    for a in areas:
        _cabi.call("kvcm_b200_route_area_detach", a)
    for sh, a in zip(shards, areas):
        sh.route_area_destroy(a)


def main_route_reference(args):
    """CPU arm of --workload route: the unsharded matchers of the oracle on a bounded sample of one rank's requests
    (the reference's index is not sharded, so there is nothing to route), all host threads."""
    from oracle import kvcm_oracle as oracle
    threads = os.cpu_count() or 1
    per_rank, sw = min(args.n_requests or 8_000_000, 2_000_000), 16
    stored, batches = _route_workload(1, per_rank)
    keys, off = batches[0]
    ox = oracle.Index()
    ox.put_uniform(stored)
    t_total, n = 0.0, 0
    while t_total < 10.0 and n < 500:
        t0 = time.perf_counter()
        ox.prefix_match_batch(keys, off, threads=threads)
        ox.sw_match_batch(keys, off, sw, threads=threads)
        t_total += time.perf_counter() - t0
        n += 1
    value = len(keys) * n / t_total
    print(json.dumps({"impl": "reference", "metric": "routed_prefix_and_window_match_token_blocks_per_s",
                      "value": value, "unit": "token-blocks/s", "n_gpus": args.gpus, "steps": n, "warmup": 0,
                      "higher_is_better": True, "dtype": "int64", "data": "synthetic",
                      "config": {"workload": "CPU restatement of prefix + sliding-window match on one unsharded index"},
                      "cpu_baseline": {"value": value, "unit": "token-blocks/s", "cores": threads, "kind": "port",
                                       "sample": "%d requests (%d keys) against an index of %d keys, %d repetitions"
                                                 % (len(off) - 1, len(keys), len(ox), n)},
                      "e2e": {"value": value, "unit": "token-blocks/s", "h2d_bytes_per_step": 0,
                              "d2h_bytes_per_step": 0}, "gpu_launches": 0}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c1", "c4", "c5", "lru", "iov", "hash", "route"])
    ap.add_argument("--n-requests", type=int, default=0,
                    help="c4: override the number of requests; route: keys per emulated rank (default 8,000,000)")
    ap.add_argument("--index-keys", type=int, default=0, help="c4: override the number of indexed keys")
    ap.add_argument("--shard-mode", default="route_peer", choices=["peer", "exchange", "route", "route_peer"],
                    help="c4 on several GPUs: probe remote shards over NVLink, or exchange keys and reduce results")
    ap.add_argument("--no-overlap", action="store_true",
                    help="c4: one stream, requests in arrival order (the earlier form of the step)")
    ap.add_argument("--match-via", default="direct", choices=["flags", "direct"],
                    help="c4 on one GPU: direct = PrefixMatch and ReverseRollSlideWindowMatch probe the index "
                         "themselves (they stop at a request's first miss and look at window ends only); flags = one "
                         "BatchGet per key, then both matchers over the flag bytes (measured: 4.42 ms per step "
                         "against 3.21: beside the hash kernels the look-up of every key costs more than it saves)")
    ap.add_argument("--long-fraction", type=str, default=None,
                    help="c4: requests at least this fraction of the longest form the head that gets its own stream "
                         "(default 0.3; 0.7 for the routed shard modes, whose head is routed after the rest)")
    ap.add_argument("--head-priority", type=int, default=1, help="c4: 1 = the head's stream has high priority")
    ap.add_argument("--head-cap", type=str, default=None,
                    help="c4: hashing warps per SM of the long head (default 2 on one GPU, 4 in the routed modes)")
    ap.add_argument("--rest-cap", type=int, default=3, help="c4: hashing warps per SM of the rest")
    ap.add_argument("--rest-chunks", type=int, default=1,
                    help="c4 on one GPU or with peer loads: streams the requests behind the long head are spread over")
    ap.add_argument("--request-tokens", type=int, default=0, help="hash: tokens per request (default 20970)")
    ap.add_argument("--n-configs", type=int, default=0, help="lru: quota points per GPU (default 148)")
    ap.add_argument("--instances", type=int, default=1,
                    help="lru: instances that share each quota (requests go to them round-robin; group-rough eviction)")
    ap.add_argument("--policy", default="lru", choices=["lru", "leaf_aware_lru", "random_lru"],
                    help="lru: the eviction policy of the sweep (eviction_policy_type)")
    ap.add_argument("--no-prefix", action="store_true", help="skip the prefix-match side measurement")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-staging leg (profiling runs)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--extras", default="auto", choices=["auto", "none", "all"],
                    help="default workload only: the other configurations measured after the headline and printed "
                         "as keys of the same line.  auto = the Llama-70B/TP8 slice (c3) and the sharded window "
                         "match (window_match) at every GPU count, the mixed replay (mixed_replay) at 8 GPUs; "
                         "all = the three of them at any GPU count; none = the headline alone (profiling runs)")
    ap.add_argument("--n-blocks", type=int, default=0, help="override the number of transfer blocks (small cases)")
    ap.add_argument("--pool-pages", type=int, default=0, help="override the pages per pool (small cases)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":  # CPU arms: rank 0 alone works, the other ranks leave at once
        if rank != 0:
            return
        arms = {"c1": lambda: main_prefix(args, None), "c4": lambda: main_window_reference(args),
                "c5": lambda: main_replay_reference(args), "lru": lambda: main_lru_reference(args),
                "iov": lambda: main_iov_reference(args), "hash": lambda: main_hash_reference(args),
                "route": lambda: main_route_reference(args)}
        if args.workload in arms:
            arms[args.workload]()
        else:
            main_reference(args, transfer_cfg(args), rank)
        return

    ctx = Ctx()
    try:
        if args.workload == "c1":
            main_prefix(args, ctx)
        elif args.workload == "route":
            if rank == 0:
                main_route(args, rank)
        elif args.workload in ("lru", "iov", "hash"):
            {"lru": main_lru, "iov": main_iov, "hash": main_hash}[args.workload](args, ctx)
        elif args.workload in ("c4", "c5"):
            line = (run_window if args.workload == "c4" else run_replay)(args, ctx)
            if rank == 0:
                print(json.dumps(line))
        else:
            main_b200(args, transfer_cfg(args), ctx)
    finally:
        ctx.close()


def transfer_cfg(args):
    cfg = dict(WORKLOADS[args.workload])
    cfg["full_size"] = not (args.n_blocks or args.pool_pages)
    if args.n_blocks:
        cfg["n_blocks"] = args.n_blocks
    if args.pool_pages:
        cfg["pool_pages"] = args.pool_pages
    if not cfg["full_size"]:
        cfg["desc"] += " [REDUCED for profiling: %d blocks, %d pages per pool]" % (cfg["n_blocks"], cfg["pool_pages"])
    return cfg


def main_b200(args, cfg, ctx):
    """The default line: the headline transfer workload, then - with inputs of the earlier parts freed - the other
    configurations as extra keys of the same line (every rank takes part in each; rank 0 prints)."""
    import gc

    import torch
    t_start = time.perf_counter()
    line = run_transfer(args, cfg, ctx, with_e2e=not args.no_e2e)
    seconds = {"headline": round(time.perf_counter() - t_start, 1)}

    def freed():
        gc.collect()
        torch.cuda.empty_cache()

    freed()
    if ctx.world == 1 and not args.no_cpu and not args.no_prefix:
        t0 = time.perf_counter()
        threads = os.cpu_count() or 1
        pm, data = run_prefix_gpu(ctx.device, 20, 3)
        pm["cpu_baseline"] = prefix_cpu_baseline(data, threads)
        line["prefix_match"] = pm
        seconds["prefix_match"] = round(time.perf_counter() - t0, 1)
        freed()
    extras = args.extras if args.workload == "c2" and cfg["full_size"] else "none"
    if extras != "none":
        t0 = time.perf_counter()
        c3 = run_transfer(args, dict(WORKLOADS["c3"], full_size=True), ctx, with_e2e=not args.no_e2e, with_cpu=False)
        line["c3"] = extra_of(c3)
        seconds["c3"] = round(time.perf_counter() - t0, 1)
        del c3
        freed()
        t0 = time.perf_counter()
        wm = run_window(args, ctx)
        if wm is not None:
            line["window_match"] = extra_of(wm)
            if ctx.world == 1 and not args.no_cpu:
                line["window_match"]["cpu_baseline"] = window_cpu_baseline(65536, os.cpu_count() or 1, budget_s=6.0)[2]
        seconds["window_match"] = round(time.perf_counter() - t0, 1)
        del wm
        freed()
        if extras == "all" or ctx.world == 8:
            t0 = time.perf_counter()
            mr = run_replay(args, ctx)
            if mr is not None:
                line["mixed_replay"] = extra_of(mr)
            seconds["mixed_replay"] = round(time.perf_counter() - t0, 1)
            del mr
            freed()
    line["wall_seconds_by_part"] = seconds
    if ctx.rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
