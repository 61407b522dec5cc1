#!/usr/bin/env python
"""Benchmark of the AMO-BQ feature-cache hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one AMO-BQ G32 decode of the pre-quantised codes of a bf16 tensor
[128, 446, 768] (43.8 M values) into a preallocated bf16 buffer -- the
configuration the headline metric is quoted on.  Prints ONE JSON line.

* ``value``     device-resident decode throughput in algorithmic GB/s
                (1 + 3/G + 2 bytes per value, GB = 1e9), CUDA events over exactly
                K launches on the launching stream; four input/output sets are
                rotated so that every launch reads and writes memory that is not
                in L2 (542 MB footprint vs 126 MB of L2).
* ``roofline``  the same bytes / average launch time against the measured HBM
                copy bandwidth in MEASURED_PEAKS.json.
* ``e2e``       the same metric through the public reader API, on the sharded-cache
                configuration: ONE cache of 65,536 samples [446, 768] written with 8 shards by the
                ranks of the node together, read by ``ZeroCopyTensorStreamer(prefix, rank=r,
                world_size=N)`` from host memory -> H2D -> decode, with a device->host read of a
                completion word every batch.  At least 200 batches are timed, from a fresh
                pass, so that the ring's prefill lies inside the timed region.
* ``streamer``  the other reader modes on the same cache (random order, staging copies,
                ``FeatureCacheDataset.iter_batches``) and the writer's rate.
* ``kernels``   (1 GPU only) the other kernels of the path on their benchmark shapes: the encoder
                on bf16 [256,1024,1024] and the fused dequantise + GEMM on 8192 x 14336 x 4096.
* ``cpu_baseline``  the C port of the reference's CPU decode (oracle/) on the host
                cores of this box, on a bounded sample; ``cpu_baseline_torch`` the reference's
                own PyTorch expression; ``reference_triton`` the reference's Triton kernels on this GPU.
* ``--impl reference``  times the CPU port alone, each step one decode of the same
                workload, with all host threads.

Multi-GPU (torchrun, one rank per GPU): shards are independent, every rank runs
the same per-GPU work on its own shards (weak scaling), no data-path collective.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPE = (128, 446, 768)
G = 32
METRIC = "amo_bq_g32_dequant_throughput"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
BYTES_PER_SAMPLE = SHAPE[1] * SHAPE[2] + 3 * (SHAPE[1] * SHAPE[2] // G)     # 374,640 compressed bytes cross PCIe per sample
C4_SAMPLES, C4_SHARDS = 65536, 8
# dram__bytes_read.sum + dram__bytes_write.sum of one isolated launch of this workload,
# from an ncu capture of this kernel on a B200: 48.03 MB read + 35.9 MB written.
DRAM_TRAFFIC_PER_LAUNCH = 83.9e6
TRAFFIC_SOURCE = "profiles/decompress_v8_kernel_G32_128x446x768.md"
TRAFFIC_NOTE = ("bytes per launch from one ncu capture: reads 48.03 MB = algorithmic reads; of the 87.69 MB stored only "
                "35.9 MB reach DRAM inside an isolated launch, the rest is written back from L2 afterwards")


def algorithmic_bytes(numel: int, g: int) -> float:
    return numel * (1.0 + 3.0 / g + 2.0)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            j = json.loads(p.read_text())
            return float(j["bf16_tflops_sustained"]), float(j["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1400.0, 1590.0, "fallback"


def workload_config(world: int, **extra) -> dict:
    """The ``config`` both arms print (same keys and values, so that the two lines describe one workload)."""
    numel = int(np.prod(SHAPE))
    cfg = {"workload": "AMO-BQ G32 decode of the codes of a bf16 [128,446,768] tensor (N(0,1) x lognormal(0,0.5) per channel, "
                       "0.1 % outliers x 20, balanced preset) into a preallocated buffer",
           "group_size": G, "values_per_step_per_gpu": numel, "algorithmic_bytes_per_step": algorithmic_bytes(numel, G),
           "parallelism": f"{world} independent replicas, one per GPU, no collective"}
    cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------- synthetic data

FEATURE_CHUNK = 256


def feature_chunk(device, seed: int, chunk: int) -> torch.Tensor:
    """Samples [256 * chunk, 256 * chunk + 256) of the synthetic feature stream `seed`: N(0,1) times a per-channel
    lognormal(0, 0.5) scale, 0.1 % of the entries multiplied by 20, bf16 [256, 446, 768].  Every chunk has its own
    generator state, so any rank can regenerate any part of the stream."""
    gch = torch.Generator(device=device).manual_seed(1_000_003 * seed + 17)
    ch = torch.exp(0.5 * torch.randn(SHAPE[2], generator=gch, device=device))
    gen = torch.Generator(device=device).manual_seed(1_000_003 * seed + 1000 + chunk)
    out = torch.empty((FEATURE_CHUNK,) + SHAPE[1:], dtype=torch.bfloat16, device=device)
    for b in range(0, FEATURE_CHUNK, 64):
        v = torch.randn((64,) + SHAPE[1:], generator=gen, device=device) * ch
        mask = torch.rand(v.shape, generator=gen, device=device) < 0.001
        out[b:b + 64] = torch.where(mask, 20 * v, v).to(torch.bfloat16)
    return out


def feature_slice(device, seed: int, first: int, n: int) -> torch.Tensor:
    """Samples [first, first + n) of feature stream `seed`."""
    parts = []
    for c in range(first // FEATURE_CHUNK, (first + n - 1) // FEATURE_CHUNK + 1):
        lo, hi = max(first, c * FEATURE_CHUNK), min(first + n, (c + 1) * FEATURE_CHUNK)
        parts.append(feature_chunk(device, seed, c)[lo - c * FEATURE_CHUNK:hi - c * FEATURE_CHUNK])
    return parts[0] if len(parts) == 1 else torch.cat(parts)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while a region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        fd, self.path = tempfile.mkstemp(prefix="tcb_clocks_", suffix=".csv")
        os.close(fd)
        self.out = open(self.path, "w")
        self.proc = subprocess.Popen([exe, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                      "-i", str(self.gpu_index)], stdout=self.out, stderr=subprocess.DEVNULL)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except (ValueError, IndexError):
            pass
    return local_index


# --------------------------------------------------------------------------- CPU

def host_codes(numel: int, g: int, seed: int):
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 256, numel, dtype=np.uint8)
    zp = rng.integers(0, 256, numel // g, dtype=np.uint8)
    s = torch.exp(torch.rand(numel // g) * 6.0 - 7.0).to(torch.bfloat16)
    return q, s, zp


def cpu_decode_rate(numel: int, g: int, budget_s: float, max_reps: int, nthreads: int):
    """Sustained rate of the C port of the reference CPU decode; returns (GB/s, reps, seconds)."""
    from oracle import amo_oracle as orc

    q, s, zp = host_codes(numel, g, 0)
    s = s.view(torch.int16).numpy().view(np.uint16)
    out = np.empty(numel, np.uint16)
    orc.decompress(q, s, zp, g, nthreads=nthreads, out=out)  # warm-up, page-faults the output
    reps, t_start = 0, time.perf_counter()
    while reps < max_reps and time.perf_counter() - t_start < budget_s:
        orc.decompress(q, s, zp, g, nthreads=nthreads, out=out)
        reps += 1
    spent = time.perf_counter() - t_start
    return algorithmic_bytes(numel, g) * reps / spent / 1e9, reps, spent


def cpu_torch_baseline(numel: int, g: int):
    """The reference's OWN CPU path: dequantize_int8_amo_bq(..., out_buffer=) of the unmodified package on CPU tensors
    (src/tensorcache/codec.py:953-966), best of 5.  Needs baseline/_ref (see baseline/install_ref.py)."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "tensorcache").is_dir():
        return {"unavailable": "baseline/_ref/tensorcache is absent (python baseline/install_ref.py puts the reference package there)"}
    sys.path.insert(0, str(ref_dir))
    try:
        from tensorcache.codec import dequantize_int8_amo_bq as ref_decode
    except Exception as e:   # noqa: BLE001
        return {"unavailable": f"the reference package does not import here: {e}"}
    finally:
        sys.path.remove(str(ref_dir))
    q, s, zp = host_codes(numel, g, 0)
    q, zp = torch.from_numpy(q), torch.from_numpy(zp)
    out = torch.empty(SHAPE, dtype=torch.bfloat16)
    ref_decode(q, s, zp, SHAPE, g, out_buffer=out)
    best = float("inf")
    for _ in range(5):
        t0 = time.perf_counter()
        ref_decode(q, s, zp, SHAPE, g, out_buffer=out)
        best = min(best, time.perf_counter() - t0)
    return {"value": algorithmic_bytes(numel, g) / best / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "reference",
            "ms_per_decode": best * 1e3,
            "sample": "best of 5 decodes of the full [128,446,768] G32 workload by the reference's dequantize_int8_amo_bq on CPU "
                      f"tensors with out_buffer, torch.get_num_threads() = {torch.get_num_threads()}"}


def cpu_reference_streamer(prefix: str, first_batch_bits, max_batches: int = 32):
    """The reference's OWN reader on the host: the unmodified ZeroCopyTensorStreamer(device="cpu") (src/tensorcache/streamer.py:334-372)
    over shard 0 of the cache THIS build's writer produced, contiguous order.  Also an interoperability check: its first
    batch must carry the bits this build's reader delivered for the same rows."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "tensorcache").is_dir():
        return {"unavailable": "baseline/_ref/tensorcache is absent (python baseline/install_ref.py puts the reference package there)"}
    sys.path.insert(0, str(ref_dir))
    try:
        from tensorcache.streamer import ZeroCopyTensorStreamer as RefStreamer
    except Exception as e:   # noqa: BLE001
        return {"unavailable": f"the reference package does not import here: {e}"}
    finally:
        sys.path.remove(str(ref_dir))
    # under torchrun OMP_NUM_THREADS is 1; give the reference this rank's share of the host cores for the leg
    had = torch.get_num_threads()
    share = max(1, (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
                // max(1, int(os.environ.get("LOCAL_WORLD_SIZE") or os.environ.get("WORLD_SIZE") or 1)))
    torch.set_num_threads(max(had, share))
    try:
        st = RefStreamer(prefix, batch_size=SHAPE[0], device="cpu", shuffle=False, shard_idx=0)
        n, same, t0 = 0, None, time.perf_counter()
        for k, batch in enumerate(st):
            if k == 0 and first_batch_bits is not None:
                same = bool(torch.equal(batch.view(torch.int16), first_batch_bits))
            n += int(batch.shape[0])
            if k + 1 >= max_batches:
                break
        spent = time.perf_counter() - t0
        st.close()
    except Exception as e:   # noqa: BLE001
        torch.set_num_threads(had)
        return {"unavailable": f"the reference reader failed on this cache: {type(e).__name__}: {e}"}
    used = torch.get_num_threads()
    torch.set_num_threads(had)
    return {"samples_per_s": n / spent, "batches": max_batches, "cores": used,
            "first_batch_bit_equal_with_this_build": same,
            "note": "unmodified reference ZeroCopyTensorStreamer(device='cpu', shuffle=False, shard_idx=0) over the cache written here"}


def run_reference_arm(args):
    """CPU port of the reference decode, all host threads; step = one decode of the full workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import amo_oracle as orc

    nthreads = orc.default_threads()
    numel = int(np.prod(SHAPE))
    n_sets = 2  # two full [128, 446, 768] workloads (271 MB together), visited alternately
    sets = []
    for i in range(n_sets):
        q, s, zp = host_codes(numel, G, i)
        sets.append((q, s.view(torch.int16).numpy().view(np.uint16), zp, np.empty(numel, np.uint16)))
    t_warm, i = time.perf_counter(), 0
    while i < max(args.warmup, n_sets) or time.perf_counter() - t_warm < 1.0:   # at least a second of warm-up
        q, s, zp, out = sets[i % n_sets]
        orc.decompress(q, s, zp, G, nthreads=nthreads, out=out)
        i += 1
    t0 = time.perf_counter()
    for i in range(args.steps):
        q, s, zp, out = sets[i % n_sets]
        orc.decompress(q, s, zp, G, nthreads=nthreads, out=out)
    dt = time.perf_counter() - t0
    value = algorithmic_bytes(numel, G) * args.steps / dt / 1e9
    sample = f"each step decodes the full [128,446,768] workload ({numel} values) with {nthreads} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8->bf16 (fp32 arithmetic)", "data": "synthetic",
        "config": workload_config(args.gpus),
        "arm_note": "C port of the reference's CPU decode on this box's host cores (the reference is Python / PyTorch; its own "
                    "expression is timed as cpu_baseline_torch in the other arm's line); host wall clock, inputs in host memory",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": nthreads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# --------------------------------------------------------------------------- GPU: cache + readers

def shared_scratch(rank: int, barrier, need_bytes: int):
    """A directory in memory-backed storage that every rank of the node sees, and whether it can hold `need_bytes`."""
    tag = os.environ.get("MASTER_PORT", "0") + "_" + os.environ.get("TORCHELASTIC_RUN_ID", "solo")
    base = "/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir()
    path = os.path.join(base, f"tcb_bench_{tag}")
    if rank == 0:
        shutil.rmtree(path, ignore_errors=True)
        os.makedirs(path, exist_ok=True)
    barrier()
    try:
        free = shutil.disk_usage(path).free
    except OSError:
        free = 0
    avail = None
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    avail = int(line.split()[1]) * 1024
    except OSError:
        pass
    roomy = free > need_bytes * 1.15 and (avail is None or avail > need_bytes * 2.2)
    return path, roomy


def write_sharded_cache(tc, prefix: str, total: int, n_shards: int, rank: int, world: int, device, barrier):
    """All ranks fill ONE `n_shards`-way cache of `total` samples.  One rank: the reference's own call,
    FeatureCacheWriter(prefix, total, ..., num_shards=n_shards).  Several ranks: rank r writes the shards i with
    i % world == r through FeatureCacheWriter.for_shard (all of them opened before the first append), rank 0 adds the
    manifest.  The rank's samples are generated on the device BEFORE the clock starts; the clock runs from before the
    writer(s) are opened until the last one is closed.  Returns (samples/s of this rank, spot-check)."""
    kw = dict(group_size=G, amo_bq=True, amo_mode="balanced")
    base, rem = divmod(total, n_shards)
    sizes = [base + (1 if i < rem else 0) for i in range(n_shards)]
    offsets = np.cumsum([0] + sizes[:-1])
    mine = list(range(rank, n_shards, world))
    BLOCK = 2048   # samples per append call (1.4 GB of bf16): eight 256-sample encode chunks in flight behind one another
    data = {}
    for i in mine:
        buf = torch.empty((sizes[i], SHAPE[1], SHAPE[2]), dtype=torch.bfloat16, device=device)
        for pos in range(0, sizes[i], BLOCK):
            n = min(BLOCK, sizes[i] - pos)
            buf[pos:pos + n] = feature_slice(device, 4, int(offsets[i]) + pos, n)
        data[i] = buf
    torch.cuda.synchronize(device)
    barrier()
    written = sum(sizes[i] for i in mine)
    t0 = time.perf_counter()
    if world == 1:
        w = tc.FeatureCacheWriter(prefix, total, SHAPE[1], SHAPE[2], num_shards=n_shards, **kw)
        for i in mine:
            for pos in range(0, sizes[i], BLOCK):
                w.append(data[i][pos:pos + BLOCK])
        w.close()
    else:
        writers = {i: tc.FeatureCacheWriter.for_shard(prefix, i, total, SHAPE[1], SHAPE[2], n_shards, **kw) for i in mine}
        for i in mine:
            for pos in range(0, sizes[i], BLOCK):
                writers[i].append(data[i][pos:pos + BLOCK])
            writers[i].close()
    spent = time.perf_counter() - t0
    data.clear()
    torch.cuda.empty_cache()
    barrier()
    if rank == 0 and world > 1:
        tc.FeatureCacheWriter.write_manifest(prefix, total, SHAPE[1], SHAPE[2], n_shards, **kw)
    barrier()
    # spot check: the first 256 rows of every shard this rank wrote against compress() of the regenerated samples
    checked, ok = 0, True
    for i in range(rank, n_shards, world):
        n = min(256, sizes[i])
        x = feature_slice(device, 4, int(offsets[i]), n)
        q, s, zp, _ = tc.compress(x, "balanced", G)
        gps = SHAPE[1] * SHAPE[2] // G
        fq = np.fromfile(f"{prefix}_shard{i}_int8.bin", dtype=np.uint8, count=n * SHAPE[1] * SHAPE[2])
        fs = np.fromfile(f"{prefix}_shard{i}_scales.bin", dtype=np.uint16, count=n * gps)
        fz = np.fromfile(f"{prefix}_shard{i}_zp.bin", dtype=np.uint8, count=n * gps)
        ok = ok and np.array_equal(fq, q.cpu().numpy()) and np.array_equal(fz, zp.cpu().numpy()) and \
            np.array_equal(fs, s.cpu().view(torch.int16).numpy().view(np.uint16))
        checked += n
    return written / max(spent, 1e-9), {"rows_checked": checked, "bit_equal_with_compress": bool(ok)}


def time_batches(make_iter, device, steps: int, warmup: int, barrier):
    """Seconds for `steps` batches of a reader, with a D2H read of a completion word every batch.  The clock starts
    BEFORE a fresh pass begins (the ring's prefill is inside the timed region); when a pass ends a new one starts."""
    token = torch.empty(16, dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream(device)

    def consume(n):
        done = 0
        while done < n:
            for batch in make_iter():
                token.copy_(batch.view(-1)[-16:], non_blocking=True)  # device -> host, ordered after the decode
                stream.synchronize()
                done += 1
                if done == n:
                    break
        return done

    consume(warmup)
    torch.cuda.synchronize(device)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    consume(steps)
    ev1.record()
    torch.cuda.synchronize(device)
    barrier()
    return ev0.elapsed_time(ev1) / 1e3, token.numel() * 2


# --------------------------------------------------------------------------- GPU: the other kernels of the path

def time_calls(fn, steps: int, warmup: int, device):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize(device)
    return ev0.elapsed_time(ev1) / 1e3 / steps


def student_t_tensor(device, gen, B, R, C):
    """bf16 [B, R, C]: Student-t (nu = 4) values times a per-channel lognormal(0, 1) scale."""
    ch = torch.exp(torch.randn(C, generator=gen, device=device))
    x = torch.empty((B, R, C), dtype=torch.bfloat16, device=device)
    for b in range(0, B, 32):
        n = min(32, B - b)
        z = torch.randn((n, R, C), generator=gen, device=device)
        wv = torch.randn((4, n, R, C), generator=gen, device=device)
        x[b:b + n] = (z / torch.sqrt((wv * wv).sum(0) / 4) * ch).to(torch.bfloat16)
        del z, wv
    return x


# thread instructions per value the encoders execute, from the ncu captures under profiles/ (issue-slot bound of the ALU work)
ENCODER_INSTR_PER_VALUE = {"fast": 14.3 * 16 + 10, "balanced": 14.3 * 32 + 10, "accurate": 14.3 * 48 + 10, "max": 14.3 * 64 + 10,
                           "quality": 1629.0}


def alu_estimate(mode: str, sm_mhz: float, sms: int = 148):
    """Values/s at which every issue slot of the GPU would be busy with this mode's instructions."""
    per_value = ENCODER_INSTR_PER_VALUE.get(mode)
    if not per_value or not sm_mhz:
        return None
    return sms * 4 * 32 * sm_mhz * 1e6 / per_value / 1e9


def reference_cpu_compress_c0(tc, device):
    """The reference's OWN CPU encoder (unmodified package under baseline/_ref, src/tensorcache/codec.py:774-893) on the
    correctness configuration, a bf16 [16,446,768] batch of the seed-0 feature stream, balanced G32; and whether this build's
    GPU encoder returns the same codes, scale bits and zero points for it."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "tensorcache").is_dir():
        return {"unavailable": "baseline/_ref/tensorcache is absent"}
    sys.path.insert(0, str(ref_dir))
    try:
        import tensorcache as ref
    except Exception as e:   # noqa: BLE001
        return {"unavailable": f"the reference package does not import here: {e}"}
    finally:
        sys.path.remove(str(ref_dir))
    x = feature_slice(device, 0, 0, 16)
    xc = x.cpu()
    t0 = time.perf_counter()
    q, s, zp, _ = ref.compress(xc, mode="balanced", group_size=G)
    spent = time.perf_counter() - t0
    q2, s2, zp2, _ = tc.compress(x, "balanced", G)
    same = bool(torch.equal(q.view(-1), q2.cpu().view(-1)) and torch.equal(s.view(torch.int16).view(-1), s2.cpu().view(torch.int16).view(-1))
                and torch.equal(zp.view(-1), zp2.cpu().view(-1)))
    return {"gvalues_per_s": xc.numel() / spent / 1e9, "ms": spent * 1e3, "cores": torch.get_num_threads(),
            "bit_equal_with_this_build": same, "note": "one run of the reference's compress() on CPU tensors, bf16 [16,446,768]"}


def kernels_section(tc, device, gpu_index):
    """Throughput of the encoder (bf16 [256,1024,1024], three modes x G16 / G32) and of the fused dequantise + GEMM
    (X [8192,4096] x AMO-BQ W [14336,4096]) with the SM clock sampled over each region."""
    from tensorcache_b200.fused_linear import check_device_status

    out = {"compress": {}, "fused_linear": None}
    gen = torch.Generator(device=device).manual_seed(2)
    x = student_t_tensor(device, gen, 256, 1024, 1024)
    hbm, _ = peaks()
    for mode in ("fast", "balanced", "quality"):
        for g in ((16, 32, 128) if mode == "balanced" else (16, 32)):   # G128: the two-lanes-per-group kernel
            steps = 8 if mode == "quality" else 30
            sampler = ClockSampler(gpu_index)
            sampler.start()
            sec = time_calls(lambda: tc.compress(x, mode, g), steps, 3, device)
            clocks = sampler.stop()
            gv = x.numel() / sec / 1e9
            est = alu_estimate(mode, clocks.get("sm_mhz") or 1965.0)
            out["compress"][f"{mode}_g{g}"] = {
                "gvalues_per_s": gv, "ms": sec * 1e3, "steps": steps, "algorithmic_gbs": gv * (3.0 + 3.0 / g),
                "frac_of_hbm": gv * (3.0 + 3.0 / g) / hbm,
                "alu_estimate": None if est is None else {
                    "gvalues_per_s_if_every_issue_slot_were_busy": est, "frac": gv / est,
                    "thread_instructions_per_value": ENCODER_INSTR_PER_VALUE[mode]},
                "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}
    out["compress"]["reference_cpu_c0_balanced_g32"] = reference_cpu_compress_c0(tc, device)
    out["compress"]["note"] = ("bf16 [256,1024,1024] Student-t(4) x lognormal(0,1) per channel; the encoders are ALU-bound (an exact division "
                               "and ~14 thread instructions per value and candidate), so the HBM fraction is low by construction")
    del x
    torch.cuda.empty_cache()
    gen = torch.Generator(device=device).manual_seed(3)
    M, N, K = 8192, 14336, 4096
    w = (0.02 * torch.randn((N, K), generator=gen, device=device)).to(torch.bfloat16)
    xx = torch.randn((M, K), generator=gen, device=device).to(torch.bfloat16)
    wq, ws, wzp, _ = tc.compress(w, "balanced", G)
    wq = wq.view(N, K)
    del w
    sustained, burst, kind = tensor_peak()
    fl = {}
    for label, steps in (("burst", 20), ("long", 1500)):
        sampler = ClockSampler(gpu_index)
        sampler.start()
        sec = time_calls(lambda: tc.fused_dequant_matmul(xx, wq, ws, wzp, None, G), steps, 3, device)
        clocks = sampler.stop()
        check_device_status()
        tf = 2.0 * M * N * K / sec / 1e12
        fl[label] = {"tflops": tf, "ms": sec * 1e3, "launches": steps, "frac_of_burst": tf / burst, "frac_of_sustained": tf / sustained,
                     "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}
    # The accuracy oracle's expression at full size on the host: fp32 dequantise-then-matmul on CPU tensors (one run), and
    # the relative Frobenius error of the kernel's bf16 result against it.
    try:
        y = tc.fused_dequant_matmul(xx, wq, ws, wzp, None, G)
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        w32 = ((wq.cpu().float().view(N, K // G, G) - wzp.cpu().float().view(N, K // G, 1)) * ws.cpu().float().view(N, K // G, 1)).view(N, K)
        ref = xx.cpu().float() @ w32.T
        spent = time.perf_counter() - t0
        yc = y.cpu().float()
        fl["reference_cpu_fp32"] = {"tflops": 2.0 * M * N * K / spent / 1e12, "ms": spent * 1e3, "cores": torch.get_num_threads(),
                                    "rel_frobenius_error_of_the_kernel": float((yc - ref).norm() / ref.norm()),
                                    "note": "fp32 dequantise-then-matmul of the same operands by torch on the host (one run, dequantisation included)"}
        del y, w32, ref, yc
    except Exception as e:   # noqa: BLE001  (host memory: the leg needs about 1.5 GB)
        fl["reference_cpu_fp32"] = {"unavailable": f"{type(e).__name__}: {e}"}
    fl["workload"] = f"X[{M},{K}] bf16 (N(0,1)) x AMO-BQ balanced G32 W[{N},{K}] (N(0, std 0.02)) -> bf16 [{M},{N}]"
    fl["peaks"] = {"bf16_tflops_burst": burst, "bf16_tflops_sustained": sustained, "kind": kind}
    fl["note"] = ("'burst' is 20 launches timed alone (compare with the burst peak), 'long' 1500 launches during which the GPU settles under "
                  "its power cap (compare with the sustained peak)")
    out["fused_linear"] = fl
    del xx, wq, ws, wzp
    torch.cuda.empty_cache()
    return out


def run_reference_triton(args):
    """The reference's own Triton kernels on this GPU (decode of [128,446,768], balanced G32 encode of [256,1024,1024],
    FusedDequantLinear on 14336 x 8192 x 4096 signed codes), from the unmodified package under baseline/_ref.  Bench only."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "tensorcache").is_dir():
        print(json.dumps({"unavailable": "baseline/_ref/tensorcache is absent"}))
        return 0
    sys.path.insert(0, str(ref_dir))
    import tensorcache as ref
    from tensorcache import codec as rcodec, fused_ops as rfused

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    res = {"triton": getattr(__import__("triton"), "__version__", "?"), "has_triton": bool(getattr(rcodec, "HAS_TRITON", False))}
    # decode
    x = feature_slice(device, 1, 0, 128)
    q, s, zp, shape = ref.compress(x, mode="balanced", group_size=G)
    out = torch.empty(SHAPE, dtype=torch.bfloat16, device=device)
    sec = time_calls(lambda: rcodec.dequantize_int8_amo_bq(q, s, zp, SHAPE, G, out_buffer=out), 200, 20, device)
    res["decode_g32"] = {"gbs": algorithmic_bytes(x.numel(), G) / sec / 1e9, "us": sec * 1e6,
                         "note": "inputs of one 136 MB workload stay in L2 between the launches"}
    # encode
    gen = torch.Generator(device=device).manual_seed(2)
    big = student_t_tensor(device, gen, 256, 1024, 1024)
    sec = time_calls(lambda: ref.compress(big, mode="balanced", group_size=G), 5, 2, device)
    res["compress_balanced_g32"] = {"gvalues_per_s": big.numel() / sec / 1e9, "ms": sec * 1e3}
    del big
    torch.cuda.empty_cache()
    # fused dequant + matmul, the reference layer's own semantics: signed activation codes [14336, 4096], dense weight [8192, 4096]
    gen = torch.Generator(device=device).manual_seed(3)
    Mq, K, Nd = 14336, 4096, 8192
    layer = rfused.FusedDequantLinear(K, Nd, bias=False, group_size=G).to(device)
    a = 0.02 * torch.randn((Mq, K), generator=gen, device=device)
    blocks = a.view(-1, G)
    sc = (blocks.abs().amax(1) / 127.0).clamp(min=1e-8).to(torch.bfloat16)
    qi = torch.clamp(torch.round(blocks / sc.float().view(-1, 1)), -127, 127).to(torch.int8).view(Mq, K)
    sec = time_calls(lambda: layer(qi, sc), 3, 1, device)
    res["fused_linear"] = {"tflops": 2.0 * Mq * Nd * K / sec / 1e12, "ms": sec * 1e3,
                           "shape": "dequant(q int8 [14336,4096]) @ weight[8192,4096]^T, the reference layer's operand roles"}
    print(json.dumps(res), flush=True)
    return 0


def reference_triton_section():
    """Runs run_reference_triton in a child process (a JIT failure or a slow compile must not take the benchmark down)."""
    try:
        r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", "reference_triton"], stdout=subprocess.PIPE,
                           stderr=subprocess.PIPE, text=True, timeout=420)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's Triton kernels did not finish within 420 s"}
    for line in reversed(r.stdout.splitlines()):
        line = line.strip()
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    return {"unavailable": f"child exited with {r.returncode}: {r.stderr.strip().splitlines()[-1] if r.stderr.strip() else 'no output'}"}


def run_other_workload(args):
    """Single-GPU timings of the other kernels of the path (not the headline line):
    fused_linear: X [8192,4096] bf16 x AMO-BQ balanced G32 weight [14336,4096]  -> TFLOP/s
    compress:     bf16 [256,1024,1024] Student-t(4) x lognormal channel scale   -> Gvalues/s
                  (--mode: an AMO-BQ preset, or sym / adaptive for the symmetric codec)
    decode_any:   decode of [128,446,768] random codes at --group-size, AMO-BQ or (--mode sym) symmetric -> GB/s"""
    import tensorcache_b200 as tc
    from tensorcache_b200.fused_linear import check_device_status

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    gen = torch.Generator(device=device).manual_seed(3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.workload == "fused_linear":
        M, N, K = (int(v) for v in args.shape.split(",")) if args.shape else (8192, 14336, 4096)
        w = (0.02 * torch.randn((N, K), generator=gen, device=device)).to(torch.bfloat16)
        x = torch.randn((M, K), generator=gen, device=device).to(torch.bfloat16)
        wq, ws, wzp, _ = tc.compress(w, "balanced", args.group_size)
        wq = wq.view(N, K)
        del w
        fn = lambda: tc.fused_dequant_matmul(x, wq, ws, wzp, None, args.group_size)
        work, unit, metric = 2.0 * M * N * K / 1e12, "TFLOP/s", "fused_dequant_linear_throughput"
        cfg = {"workload": f"FusedDequantLinear X[{M},{K}] bf16 x AMO-BQ balanced G{args.group_size} W[{N},{K}] -> bf16 [{M},{N}]"}
    elif args.workload == "decode_any":
        g = args.group_size
        numel = 128 * 446 * 768 // g * g
        sym = args.mode in ("sym", "adaptive")
        sets = []
        for k in range(4):   # rotate 4 x 136 MB so that no launch finds its inputs in L2
            q = torch.randint(0, 256, (numel,), generator=gen, device=device, dtype=torch.uint8)
            sc = torch.exp(torch.rand(numel // g, generator=gen, device=device) * 6 - 8).to(torch.bfloat16)
            zp = None if sym else torch.randint(0, 256, (numel // g,), generator=gen, device=device, dtype=torch.uint8)
            sets.append((q.view(torch.int8) if sym else q, sc, zp, torch.empty(numel, dtype=torch.bfloat16, device=device)))
        it = [0]

        def fn():
            q, sc, zp, out = sets[it[0] & 3]
            it[0] += 1
            if sym:
                tc.dequantize_int8_g32(q, sc, (numel,), g, out_buffer=out)
            else:
                tc.dequantize_int8_amo_bq(q, sc, zp, (numel,), g, out_buffer=out)
        bpv = 3.0 + (2.0 if sym else 3.0) / g
        work, unit, metric = numel * bpv / 1e9, "GB/s", f"{'sym' if sym else 'amo_bq'}_g{g}_dequant_throughput"
        cfg = {"workload": f"{'symmetric' if sym else 'AMO-BQ'} G{g} decode of {numel} codes into a preallocated bf16 buffer",
               "algorithmic_bytes_per_value": bpv, "l2": "4 rotating buffer sets of 136 MB each"}
    else:
        B, R, C = (int(v) for v in args.shape.split(",")) if args.shape else (256, 1024, 1024)
        x = student_t_tensor(device, gen, B, R, C)
        fn = lambda: tc.compress(x, args.mode, args.group_size)
        work, unit, metric = x.numel() / 1e9, "Gvalues/s", f"amo_bq_compress_{args.mode}_g{args.group_size}_throughput"
        cfg = {"workload": f"AMO-BQ compress mode={args.mode} G{args.group_size} of bf16 [{B},{R},{C}]",
               "algorithmic_bytes_per_value": 3.0 + (2.0 if args.mode in ("sym", "adaptive") else 3.0) / args.group_size}
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize(device)
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    ev0.record()
    for _ in range(args.steps):
        fn()
    ev1.record()
    torch.cuda.synchronize(device)
    clocks = sampler.stop()
    if args.workload == "fused_linear":
        check_device_status()
    secs = ev0.elapsed_time(ev1) / 1e3
    value = work * args.steps / secs
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "data": "synthetic", "config": cfg,
            "gpu_launches": args.steps, "clocks": clocks}
    if args.workload == "fused_linear":
        sustained, burst, kind = tensor_peak()
        line["dtype"] = "bf16 operands (dequantised in-kernel), fp32 accumulate"
        # a timed region of well under a second runs at burst clocks: compare it with the burst peak; a long one
        # settles under the power cap and is compared with the sustained peak (both fractions are given)
        long_run = secs >= 1.0
        peak = sustained if long_run else burst
        line["roofline"] = {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                            "regime": "sustained (power-capped)" if long_run else "burst", "frac_of_sustained": value / sustained,
                            "frac_of_burst": value / burst, "peak_kind": kind, "traffic": None}
    elif args.workload == "decode_any":
        hbm, kind = peaks()
        line["dtype"] = "u8/i8 -> bf16 (fp32 arithmetic)"
        line["roofline"] = {"bound": "hbm", "achieved": value, "peak": hbm, "unit": "GB/s", "frac": value / hbm, "peak_kind": kind,
                            "traffic": None}
    else:
        hbm, kind = peaks()
        gbs = value * cfg["algorithmic_bytes_per_value"]
        est = alu_estimate(args.mode, clocks.get("sm_mhz") or 1965.0)
        line["dtype"] = "fp32 (IEEE div / rint, no FMA)"
        line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "peak_kind": kind,
                            "traffic": None, "alu_estimate_gvalues_per_s": est, "frac_of_alu_estimate": None if est is None else value / est,
                            "note": "the encoder is ALU-bound (one IEEE division and ~10 dependent fp32 operations "
                            "per value and candidate); the HBM fraction is low by construction"}
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="tcb200", choices=["tcb200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=0, help="batches timed through the readers (default and minimum: 200)")
    ap.add_argument("--cache-samples", type=int, default=0, help="samples of the sharded cache (default: 65,536, or 8,192 when memory is short)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the kernels / reference_triton / cpu_baseline_torch sections")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed decodes one by one instead of replaying CUDA graphs")
    ap.add_argument("--decode-only", action="store_true", help="skip everything but the decode loop (for profiler captures)")
    ap.add_argument("--workload", default="decode", choices=["decode", "fused_linear", "compress", "decode_any", "reference_triton"],
                    help="decode (default) is the headline metric; the others time the remaining kernels of the path")
    ap.add_argument("--shape", default="", help="fused_linear: M,N,K; compress: B,R,C (defaults: the benchmark configurations)")
    ap.add_argument("--mode", default="balanced", help="compress: AMO-BQ mode, or sym / adaptive; decode_any: sym selects the symmetric codec")
    ap.add_argument("--group-size", type=int, default=G)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "reference_triton":
        return run_reference_triton(args)
    if args.workload != "decode":
        return run_other_workload(args)

    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        print(json.dumps({"metric": METRIC, "error": "no CUDA device: this path has no CPU fallback"}))
        return 1
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()

    def reduce_over_ranks(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def max_over_ranks(x: float) -> float:
        return reduce_over_ranks(x, dist.ReduceOp.MAX)

    def pinned_h2d_rate():
        """Plain pinned-memory H2D copy rate of this rank while every other rank does the same:
        the ceiling of the reader path on this box at this number of GPUs."""
        nbytes = 256 << 20
        d = torch.empty(nbytes, dtype=torch.uint8, device=device)
        # four separately allocated source buffers: where a buffer's pages sit relative to the GPU's root port moves the rate by
        # 10 % on some boxes of the pool, and the ceiling is what the link can do, so the best buffer counts
        hosts = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in range(4)]
        d.copy_(hosts[0], non_blocking=True)
        torch.cuda.synchronize(device)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = 0.0
        for rnd in range(8):   # best of eight rounds of eight copies (single rounds vary by 15 % from box to box)
            h = hosts[rnd % len(hosts)]
            e0.record()
            for _ in range(8):
                d.copy_(h, non_blocking=True)
            e1.record()
            torch.cuda.synchronize(device)
            best = max(best, 8 * nbytes / (e0.elapsed_time(e1) / 1e3) / 1e9)
        barrier()
        # The same copies for a fixed time window, the four buffers in turn: every rank copies during the WHOLE window, so no
        # rank's figure comes from a moment at which the others had finished (best-of-rounds above can), and 1 GB of source
        # per rank is not re-read from the CPU's caches.  This is what the ranks get while all of them stream.
        window_s, copied, k = 0.6, 0, 0
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < window_s:
            d.copy_(hosts[k % len(hosts)], non_blocking=True)
            d.copy_(hosts[(k + 1) % len(hosts)], non_blocking=True)
            torch.cuda.synchronize(device)
            copied += 2 * nbytes
            k += 2
        concurrent = copied / (time.perf_counter() - t0) / 1e9
        barrier()
        return best, concurrent

    import tensorcache_b200 as tc
    from tensorcache_b200 import _lib

    L = _lib.lib()  # raises if the CUDA library is missing
    numel = int(np.prod(SHAPE))
    n_sets = 4
    sets = []
    for i in range(n_sets):
        # set 0 of rank 0 holds the codes of the benchmark tensor (feature stream 1); the other sets and ranks take other streams
        x = feature_slice(device, 1 + i + n_sets * rank, 0, SHAPE[0])
        q, s, zp, _ = tc.compress(x, "balanced", G)
        sets.append((q, s, zp, torch.empty(SHAPE, dtype=torch.bfloat16, device=device)))
        del x
    stream = torch.cuda.current_stream(device)

    # plain integers once, so that a launch costs one ctypes call and nothing else on the host
    ptrs = [(q.data_ptr(), s.data_ptr(), zp.data_ptr(), out.data_ptr()) for q, s, zp, out in sets]

    def step(i, stream_handle):
        qp, sp, zpp, op = ptrs[i % n_sets]
        rc = L.tcb_decompress_amo(qp, sp, zpp, op, numel, G, stream_handle)
        if rc != 0:
            _lib.check(rc)

    for i in range(args.warmup):
        step(i, stream.cuda_stream)
    torch.cuda.synchronize(device)

    # The K timed launches are replayed from CUDA graphs of up to GRAPH_LAUNCHES launches each (plus a
    # remainder graph), so that the host's launch rate cannot become the limit when many ranks share few cores.
    GRAPH_LAUNCHES = n_sets * 25
    graphs = {}
    if not args.no_graph:
        side = torch.cuda.Stream(device)
        for n in {min(GRAPH_LAUNCHES, args.steps), args.steps % GRAPH_LAUNCHES}:
            if n <= 0:
                continue
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                h = torch.cuda.current_stream(device).cuda_stream
                for i in range(n):
                    step(i, h)
            graphs[n] = g
        torch.cuda.synchronize(device)
        for g in graphs.values():   # one untimed replay each
            g.replay()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(physical_gpu_index(local))
    if rank == 0:
        sampler.start()
    barrier()
    torch.cuda.synchronize(device)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # Untimed launches enqueued directly ahead of the start event, with no host synchronisation in between: the GPU is
    # already decoding when the event and the K timed launches reach it, so that a short timed region (K = 20 is 0.46 ms)
    # does not contain the launch latency of its own first graph or a GPU that went idle during the barrier.
    pre_roll = 0
    while pre_roll < 100:
        if graphs:
            n = max(graphs)
            graphs[n].replay()
            pre_roll += n
        else:
            step(pre_roll, stream.cuda_stream)
            pre_roll += 1
    ev0.record(stream)
    if graphs:
        full, rest = divmod(args.steps, GRAPH_LAUNCHES)
        for _ in range(full):
            graphs[GRAPH_LAUNCHES].replay()
        if rest:
            graphs[rest].replay()
    else:
        for i in range(args.steps):
            step(i, stream.cuda_stream)
    ev1.record(stream)
    torch.cuda.synchronize(device)
    barrier()
    secs = max_over_ranks(ev0.elapsed_time(ev1) / 1e3)
    clocks = sampler.stop() if rank == 0 else None   # sampled over the timed decode loop

    bytes_per_step = algorithmic_bytes(numel, G)
    value = bytes_per_step * args.steps * world / secs / 1e9
    per_gpu = bytes_per_step * args.steps / secs / 1e9
    peak, peak_kind = peaks()
    del sets, graphs
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ the sharded cache and its readers
    e2e = streamer = pcie = c4 = None
    e2e_steps = max(200, args.e2e_steps)
    if not args.decode_only:
        want = args.cache_samples or C4_SAMPLES
        scratch, roomy = shared_scratch(rank, barrier, want * BYTES_PER_SAMPLE)
        roomy = bool(reduce_over_ranks(1.0 if roomy else 0.0, dist.ReduceOp.MIN)) if world > 1 else roomy
        total = want if (roomy or args.cache_samples) else 8192
        prefix = os.path.join(scratch, "feat")
        try:
            writer_rate, spot = write_sharded_cache(tc, prefix, total, C4_SHARDS, rank, world, device, barrier)
            spot_ok = bool(reduce_over_ranks(1.0 if spot["bit_equal_with_compress"] else 0.0, dist.ReduceOp.MIN)) if world > 1 \
                else spot["bit_equal_with_compress"]
            writer_rate_min = reduce_over_ranks(writer_rate, dist.ReduceOp.MIN)
            kw = dict(batch_size=SHAPE[0], device=str(device), rank=rank, world_size=world, all_rank_shards=True)
            times = {}
            np.random.seed(1234 + rank)
            t_pin = time.perf_counter()
            st = tc.ZeroCopyTensorStreamer(prefix, shuffle=False, **kw)          # default mode (pin_shard=None)
            t_pin = time.perf_counter() - t_pin
            default_mode = "resident (shards page-locked)" if st.pin_shard else "staging copies"
            samples_per_rank = st.num_samples
            first_bits = None
            if rank == 0 and not args.no_extras:
                for b in st:     # the first batch of shard 0, kept for the comparison with the reference's own reader
                    first_bits = b.view(torch.int16).cpu()
                    break
            times["default_contig"], d2h = time_batches(lambda: iter(st), device, e2e_steps, args.warmup, barrier)
            st.shuffle = True
            times["default_random"], _ = time_batches(lambda: iter(st), device, e2e_steps, args.warmup, barrier)
            st.close()
            st = tc.ZeroCopyTensorStreamer(prefix, shuffle=False, pin_shard=False, **kw)
            times["staging_contig"], _ = time_batches(lambda: iter(st), device, e2e_steps, args.warmup, barrier)
            st.shuffle = True
            times["staging_random"], _ = time_batches(lambda: iter(st), device, e2e_steps, args.warmup, barrier)
            st.close()
            ds = tc.FeatureCacheDataset(prefix, rank=rank, world_size=world, all_rank_shards=True)
            times["iter_batches_contig"], _ = time_batches(
                lambda: ds.iter_batches(batch_size=SHAPE[0], shuffle=False, device=str(device)), device, e2e_steps, args.warmup, barrier)
            iter_mode = "resident (shards page-locked)" if ds.pin_shard else "staging copies"
            ds.close()
            ref_reader = cpu_reference_streamer(prefix, first_bits) if (rank == 0 and not args.no_extras) else None
        finally:
            barrier()
            if rank == 0:
                shutil.rmtree(scratch, ignore_errors=True)
        times = {k: max_over_ranks(v) for k, v in times.items()}
        rate = {k: SHAPE[0] * e2e_steps * world / v for k, v in times.items()}
        mine, mine_window = pinned_h2d_rate()
        pcie = {"pinned_h2d_gbs_per_gpu_min": reduce_over_ranks(mine, dist.ReduceOp.MIN),
                "pinned_h2d_gbs_sum": reduce_over_ranks(mine, dist.ReduceOp.SUM),
                "pinned_h2d_gbs_sum_all_ranks_streaming": reduce_over_ranks(mine_window, dist.ReduceOp.SUM),
                "pinned_h2d_gbs_per_gpu_min_all_ranks_streaming": reduce_over_ranks(mine_window, dist.ReduceOp.MIN),
                "note": "plain 256 MB pinned-memory copies issued by all ranks at once (best of four source buffers re-read eight times; *_all_ranks_streaming: every rank copies for the same 0.6 s window, the four buffers in turn); the reader path moves "
                        "374,640 compressed bytes per sample over this link"}
        pcie["ceiling_samples_per_s"] = pcie["pinned_h2d_gbs_sum"] * 1e9 / BYTES_PER_SAMPLE
        # the timed region ends when the slowest rank has finished its batches (max over ranks), so with unequal
        # link shares the ceiling of `e2e` is N times the slowest rank's rate, not the sum
        pcie["ceiling_samples_per_s_max_over_ranks"] = world * pcie["pinned_h2d_gbs_per_gpu_min"] * 1e9 / BYTES_PER_SAMPLE
        pcie["samples_per_s_all_ranks_streaming"] = pcie["pinned_h2d_gbs_sum_all_ranks_streaming"] * 1e9 / BYTES_PER_SAMPLE
        pcie["samples_per_s_all_ranks_streaming_max_over_ranks"] = \
            world * pcie["pinned_h2d_gbs_per_gpu_min_all_ranks_streaming"] * 1e9 / BYTES_PER_SAMPLE
        h2d = SHAPE[0] * BYTES_PER_SAMPLE
        e2e = {"value": bytes_per_step * e2e_steps * world / times["default_contig"] / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "samples_per_s": rate["default_contig"],
               "h2d_gbs": rate["default_contig"] * BYTES_PER_SAMPLE / 1e9,
               "within_pcie_ceiling": rate["default_contig"] * BYTES_PER_SAMPLE / 1e9 <= 1.02 * pcie["pinned_h2d_gbs_sum"],
               "reader_mode": default_mode,
               "path": f"ZeroCopyTensorStreamer(prefix, batch_size=128, shuffle=False, rank=r, world_size={world}, all_rank_shards=True) "
                       f"with the default pin_shard=None over ONE {total}-sample cache of {C4_SHARDS} shards in host memory: rows -> H2D -> "
                       "decode -> D2H completion word, every batch; the clock starts before a fresh pass begins"}
        streamer = {"samples_per_s": rate, "bf16_equiv_gbs_default_contig": rate["default_contig"] * SHAPE[1] * SHAPE[2] * 2 / 1e9,
                    "default_mode": default_mode, "iter_batches_mode": iter_mode, "open_seconds_default_mode": t_pin,
                    "writer_samples_per_s_per_rank": writer_rate_min, "reference_cpu_streamer": ref_reader,
                    "samples_per_rank": samples_per_rank, "batch_size": SHAPE[0], "batches_timed": e2e_steps,
                    "note": "default_* = pin_shard=None (what a drop-in user gets); staging_* = pin_shard=False (rows copied into "
                            "page-locked staging by worker threads, the reference's scheme); iter_batches = FeatureCacheDataset.iter_batches"}
        c4 = {"samples": total, "shards": C4_SHARDS, "bytes": total * BYTES_PER_SAMPLE,
              "written_by": ("1 rank, FeatureCacheWriter(prefix, total, 446, 768, amo_bq=True, amo_mode='balanced', num_shards=8)" if world == 1
                             else f"{world} ranks, FeatureCacheWriter.for_shard for shard i on rank i % {world}, manifest by rank 0")
                            + "; samples on the device beforehand, clock from opening the writer to its close",
              "full_size": total == C4_SAMPLES, "spot_check": {"rows_per_shard": 256, "bit_equal_with_compress": spot_ok},
              "rank_to_shards": f"rank r reads the shards i with i % {world} == r (identical to shard r % 8 of the reference at 8 ranks)"}

    cpu = cpu_torch = triton_ref = kernels = None
    if rank == 0 and not args.no_cpu_baseline and not args.decode_only:
        from oracle import amo_oracle as orc

        nthreads = orc.default_threads()
        rate_cpu, reps, spent = cpu_decode_rate(numel, G, budget_s=12.0, max_reps=5000, nthreads=nthreads)
        cpu = {"value": rate_cpu, "unit": UNIT, "cores": nthreads, "kind": "port",
               "sample": f"{reps} back-to-back decodes of the full [128,446,768] G32 workload in {spent:.1f} s, "
                         f"C port of the reference CPU decode, {nthreads} threads"}
        if not args.no_extras:
            cpu_torch = cpu_torch_baseline(numel, G)
    if rank == 0 and world == 1 and not args.no_extras and not args.decode_only:
        kernels = kernels_section(tc, device, physical_gpu_index(local))
        triton_ref = reference_triton_section()
    barrier()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8->bf16 (fp32 arithmetic)", "data": "synthetic",
            "config": workload_config(world),
            "timing": {"launch": "eager" if args.no_graph else f"CUDA graphs of {min(GRAPH_LAUNCHES, args.steps)} launches",
                       "untimed_launches_enqueued_directly_before_the_start_event": pre_roll,
                       "l2_policy": f"{n_sets} rotating input/output sets ({n_sets * bytes_per_step / 1e6:.0f} MB) > 126 MB L2",
                       "cache": None if c4 is None else f"one {c4['samples']}-sample cache of {C4_SHARDS} shards "
                                                        f"({c4['bytes'] / 1e9:.1f} GB) in host memory, B = 128 per rank"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "traffic": DRAM_TRAFFIC_PER_LAUNCH, "traffic_source": TRAFFIC_SOURCE, "traffic_note": TRAFFIC_NOTE,
                         "peak_kind": peak_kind, "kernel": "decompress_v8_kernel<G32>", "us_per_launch": secs / args.steps * 1e6},
            "e2e": e2e, "streamer": streamer, "c4": c4, "pcie": pcie,
            "cpu_baseline": cpu, "cpu_baseline_torch": cpu_torch, "kernels": kernels, "reference_triton": triton_ref,
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def _run_with_clean_stdout():
    """Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line there.
    File descriptor 1 is pointed at stderr while the benchmark runs and the line goes to the real stdout."""
    sys.stdout.flush()
    real = os.dup(1)
    os.dup2(2, 1)
    buf = []

    class _Capture:
        def write(self, t):
            buf.append(t)
            return len(t)

        def flush(self):
            pass

    old = sys.stdout
    sys.stdout = _Capture()
    try:
        rc = main()
    finally:
        sys.stdout = old
        sys.stdout.flush()
        os.dup2(real, 1)
        os.close(real)
        text = "".join(buf)
        if text:
            sys.stdout.write(text if text.endswith("\n") else text + "\n")
            sys.stdout.flush()
    return rc


if __name__ == "__main__":
    sys.exit(_run_with_clean_stdout())
