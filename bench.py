#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path. Contract: `python bench.py --gpus N --steps K --warmup W` prints ONE JSON line.

Headline workload (`--workload c2`, the default): weight_quant_batch_matmul_v2 W4A16 decode, x bf16 [16, 8192],
weight int4 [8192, 28672] packed 8 per int32 along n, per-group (128) bf16 scale + offset, y bf16 [16, 28672];
HBM-bound, metric = achieved HBM GB/s on the algorithmic bytes (125.96 MB per call). One "step" is one call.

  value   device-timed throughput with every operand resident in HBM. The weight (117 MB) would fit the 126 MB L2, so
          the steps rotate over 4 distinct weight/scale/offset sets (504 MB) and every step streams from DRAM.
  e2e     the same call through the aclnn C ABI starting from HOST buffers: per step the activation x is copied from
          pinned host memory to the device and y is copied back; the quantised weight, being a static model parameter,
          is uploaded once before the timed region (its upload time is reported separately as `weight_upload_ms`).
  N > 1   one process per GPU (torchrun); the weight is sharded along n with a fixed [8192, 28672] shard per rank (weak
          scaling: the global n grows with N), x replicated, no collective on the data path. Timing = max over ranks.

`--impl reference` times the CPU restatement of the reference's golden (oracle/, numpy on all host cores) on the same
workload and prints the same line with "impl": "reference".
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, N, G = 16, 8192, 28672, 128
ALGO_BYTES = K * N // 2 + 2 * (K // G) * N * 2 + M * K * 2 + M * N * 2  # 125,960,192


def load_package():
    pkg_dir = os.path.join(ROOT, "ops-nn_b200")
    if "ops_nn_b200" in sys.modules:
        return sys.modules["ops_nn_b200"]
    spec = importlib.util.spec_from_file_location("ops_nn_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ops_nn_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (reading only)."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            pass
        mhz, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
                for name, col in (("hw_slowdown", 4), ("hw_thermal_slowdown", 5), ("sw_thermal_slowdown", 6), ("sw_power_cap", 7)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:  # noqa: BLE001
                continue
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


WORKLOAD_C2 = "c2: W4A16 decode m16 k8192 n28672 group128 bf16 scale+offset, int4 packed 8/int32 along n"


def make_inputs(torch, dev, seed, sets):
    gen = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn((M, K), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    data = []
    for _ in range(sets):
        w = torch.randint(-8, 8, (K, N), generator=gen, device=dev, dtype=torch.int32)
        words = torch.zeros((K, N // 8), dtype=torch.int32, device=dev)
        for j in range(8):
            words |= (w[:, j::8] & 0xF) << (4 * j)
        del w
        scale = (torch.rand((K // G, N), generator=gen, device=dev) * 0.015 + 0.005).to(torch.bfloat16)
        offset = (torch.rand((K // G, N), generator=gen, device=dev) * 2 - 1).to(torch.bfloat16)
        data.append((words, scale, offset))
    return x, data


def cpu_oracle_once(x_np, words_np, scale_np, offset_np):
    from oracle import wqbmm_oracle

    t0 = time.perf_counter()
    w = wqbmm_oracle.unpack_int4_words(words_np)
    y = wqbmm_oracle.weight_quant_batch_matmul(x_np, w, scale_np, offset_np, None, G)
    return time.perf_counter() - t0, y


def cpu_c_oracle_once(x_np, words_np, scale_np, offset_np, cols):
    """The plain-C restatement (oracle/c) on all host cores over the first `cols` columns; returns seconds scaled to the
    full width, or None when the C oracle is not built and cannot be built here."""
    import numpy as np

    try:
        from oracle import c_oracle

        c_oracle.lib()
    except Exception:
        return None
    threads = os.cpu_count() or 1
    u16 = lambda a: a.view(np.uint16)
    t0 = time.perf_counter()
    c_oracle.wq_w4a16_group(u16(x_np), words_np, u16(scale_np), u16(offset_np), G, 0, cols, threads=threads)
    return (time.perf_counter() - t0) * (N / cols)


def cpu_baseline_c2(x_np, words_np, scale_np, offset_np):
    """CPU baseline of the c2 workload: the faster of the numpy restatement of the reference golden (one full call, BLAS
    threads) and the C restatement (all cores, a 2048-column panel scaled to the full width)."""
    sec_np, _ = cpu_oracle_once(x_np, words_np, scale_np, offset_np)
    sec_c = cpu_c_oracle_once(x_np, words_np, scale_np, offset_np, 2048)
    use_c = sec_c is not None and sec_c < sec_np
    sec = sec_c if use_c else sec_np
    sample = ("C restatement of the reference golden, %d threads, 2048-column panel scaled x%d (numpy restatement, full call: %.2f s)"
              % (os.cpu_count() or 1, N // 2048, sec_np)) if use_c else (
        "one full call of the numpy restatement of the reference golden (%.2f s%s)"
        % (sec_np, "" if sec_c is None else "; C restatement on all cores: %.2f s" % sec_c))
    return sec, {"value": ALGO_BYTES / sec / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample}


def to_np_bf16(t):
    import ml_dtypes
    import torch

    return t.view(torch.int16).cpu().numpy().view(ml_dtypes.bfloat16)


def run_reference(args):
    """CPU arm: the oracle port of the reference golden, all host cores numpy can use, on the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ml_dtypes
    import numpy as np

    rng = np.random.default_rng(1002)
    x = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
    words = rng.integers(-2 ** 31, 2 ** 31, (K, N // 8), dtype=np.int64).astype(np.int32)
    scale = rng.uniform(0.005, 0.02, (K // G, N)).astype(np.float32).astype(ml_dtypes.bfloat16)
    offset = rng.uniform(-1, 1, (K // G, N)).astype(np.float32).astype(ml_dtypes.bfloat16)
    for _ in range(min(args.warmup, 1)):
        cpu_baseline_c2(x, words, scale, offset)
    steps = max(1, min(args.steps, 3))
    runs = [cpu_baseline_c2(x, words, scale, offset) for _ in range(steps)]
    sec = sum(r[0] for r in runs) / len(runs)
    gbs = ALGO_BYTES / sec / 1e9
    base = dict(runs[-1][1], value=gbs)
    line = {"impl": "reference", "metric": "W4A16 decode HBM GB/s (weight_quant_batch_matmul_v2, algorithmic bytes / time)",
            "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": WORKLOAD_C2},
            "cpu_baseline": base,
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


QMM_WORKLOADS = {
    # name: (batch, m, k, n, kind)
    "c1": (1, 128, 4096, 4096, "int8_kc"),
    "c3": (1, 4096, 7168, 18432, "fp8_perblock"),
    "c3i8": (1, 4096, 7168, 18432, "int8_kc"),
    "c3i8pb": (1, 4096, 7168, 18432, "int8_perblock"),  # int8 operands with the 1x128 / 128x128 fp32 scales of c3
    "c3t": (1, 4096, 7168, 18432, "fp8_perblock_t"),    # c3 with x2 stored (n,k), transposeX2 = true
    "c3i8pbt": (1, 4096, 7168, 18432, "int8_perblock_t"),
    "c1t": (1, 128, 4096, 4096, "int8_kc_t"),      # same with x2 stored (n,k) and transposeX2 = true
    "c3i8t": (1, 4096, 7168, 18432, "int8_kc_t"),
    "c4": (8, 8192, 8192, 8192, "mxfp4"),           # both operands e2m1 + e8m0/32, x2 stored (n,k) with transposeX2 = true
    "c4s": (2, 4096, 4096, 4096, "mxfp4"),          # small form of c4 (profiling)
    "c4n": (8, 8192, 8192, 8192, "mxfp4_n"),        # c4 with the weight stored (k,n): transposed into workspace by a pre-pass
    "c5": (32, 2048, 4096, 14336, "mxfp8_dq"),      # bf16 activations -> dynamic mx quant -> mxfp8 matmul + fp32 bias
    "c5s": (4, 2048, 4096, 4096, "mxfp8_dq"),
    "c5mm": (32, 2048, 4096, 14336, "mxfp8"),       # the matmul of c5 alone (activations pre-quantised)
    "c5w": (1, 65536, 4096, 14336, "mxfp8"),        # c5mm's rows against ONE weight stored (k,n): the weight is moved k-contiguous first
    "c5h": (1, 4096, 4096, 14336, "mxfp8"),         # the smallest row count at which that move is made
    "c5mmt": (32, 2048, 4096, 14336, "mxfp8_t"),    # same with the weight stored (n,k), transposeX2 = true
    "c2p": (1, 2048, 8192, 28672, "w4a16_prefill"), # the headline weight at a prefill m: dequant pre-pass + bf16 tcgen05 matmul
    "c2ps": (1, 256, 8192, 28672, "w4a16_prefill"),
    "c2m32": (1, 32, 8192, 28672, "w4a16_prefill"),  # 16 < m <= 48: the decode kernel once per 16 rows
    "c2m48": (1, 48, 8192, 28672, "w4a16_prefill"),
}


def run_qmm_workload(args):
    """Secondary workloads (`--workload c1|c3|c3i8`): aclnnQuantMatmulV5 timed on device, TFLOPS against the measured bf16
    GEMM ceiling x2 (8-bit operands) and the datasheet dense peak. Same timing discipline as the headline workload."""
    import torch

    aclnn = load_package().aclnn
    dev = torch.device("cuda", 0)
    b, m, k, n, kind = QMM_WORKLOADS[args.workload]
    gen = torch.Generator(device=dev).manual_seed(1001)
    sets = max(2, min(8, int(300e6 // (k * n)) + 1))  # rotate weights so they do not sit in L2
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    if kind.startswith("mx"):
        # batched mx workloads: the operands (>= 270 MB per call) exceed L2 by themselves, one weight set
        sets = 1
        f4 = kind.startswith("mxfp4")
        kq = k // 64
        out = torch.empty((b, m, n), dtype=torch.bfloat16, device=dev)
        rnd_scale = lambda *shape: torch.randint(124, 131, shape, generator=gen, device=dev, dtype=torch.uint8)  # noqa: E731
        if f4:
            x1 = torch.randint(0, 256, (b, m, k // 2), generator=gen, device=dev, dtype=torch.uint8)  # two e2m1 per byte
            nmaj = kind == "mxfp4_n"
            x2 = torch.randint(0, 256, (b, k, n // 2) if nmaj else (b, n, k // 2), generator=gen, device=dev, dtype=torch.uint8)
            d_x1 = aclnn.from_torch(x1, "float4_e2m1", (b, m, k), (m * k, k, 1))
            d_x2 = (aclnn.from_torch(x2, "float4_e2m1", (b, k, n), (n * k, n, 1)) if nmaj
                    else aclnn.from_torch(x2, "float4_e2m1", (b, n, k), (n * k, k, 1)))  # stored (n,k): transposeX2 = true
            s1, s2 = rnd_scale(b, m, kq, 2), (rnd_scale(b, kq, n, 2) if nmaj else rnd_scale(b, n, kq, 2))
            d_s1 = aclnn.from_torch(s1, "float8_e8m0")
            d_s2 = aclnn.from_torch(s2, "float8_e8m0")
            dout = aclnn.from_torch(out)
            call = lambda i: aclnn.quant_matmul_v5(d_x1, d_x2, d_s1, d_s2, dout, None, False, not nmaj, (1 << 32) | (1 << 16) | 32)  # noqa: E731
            nbytes = b * (m * k // 2 + n * k // 2 + (m + n) * kq * 2 + 2 * m * n)
        else:
            tb = kind == "mxfp8_t"
            x2 = torch.randn((b, n, k) if tb else (b, k, n), generator=gen, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn)
            s2 = rnd_scale(b, n, kq, 2) if tb else rnd_scale(b, kq, n, 2)
            bias = torch.randn((n,), generator=gen, device=dev, dtype=torch.float32)
            x1q = torch.empty((b, m, k), dtype=torch.uint8, device=dev)
            s1 = torch.empty((b, m, kq, 2), dtype=torch.uint8, device=dev)
            d_x1 = aclnn.from_torch(x1q, "float8_e4m3fn")
            d_s1 = aclnn.from_torch(s1, "float8_e8m0")
            d_x2, d_s2, d_bias, dout = aclnn.from_torch(x2), aclnn.from_torch(s2, "float8_e8m0"), aclnn.from_torch(bias), aclnn.from_torch(out)
            act = torch.randn((b, m, k), generator=gen, device=dev, dtype=torch.bfloat16)
            act.view(-1)[torch.randint(0, act.numel(), (act.numel() // 1000,), generator=gen, device=dev)] *= 50  # 0.1 % outliers
            d_act = aclnn.from_torch(act)
            aclnn.dynamic_mx_quant(d_act, d_x1, d_s1, "float8_e4m3fn")
            mm = lambda: aclnn.quant_matmul_v5(d_x1, d_x2, d_s1, d_s2, dout, d_bias, False, tb, (1 << 32) | (1 << 16) | 32)  # noqa: E731
            if kind == "mxfp8_dq":
                def call(i):
                    aclnn.dynamic_mx_quant(d_act, d_x1, d_s1, "float8_e4m3fn")
                    mm()
                nbytes = b * (2 * m * k + m * k + k * n + (m + n) * kq * 2 + 2 * m * n)
            else:
                call = lambda i: mm()  # noqa: E731
                nbytes = b * (m * k + k * n + (m + n) * kq * 2 + 2 * m * n)
    elif kind == "w4a16_prefill":
        sets = 1  # the packed weight (117 MB) plus its dequantised copy (470 MB) exceed L2 by themselves
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        x = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        w = torch.randint(-8, 8, (k, n), generator=gen, device=dev, dtype=torch.int32)
        words = torch.zeros((k, n // 8), dtype=torch.int32, device=dev)
        for j in range(8):
            words |= (w[:, j::8] & 0xF) << (4 * j)
        del w
        scale = (torch.rand((k // 128, n), generator=gen, device=dev) * 0.015 + 0.005).to(torch.bfloat16)
        offset = (torch.rand((k // 128, n), generator=gen, device=dev) * 2 - 1).to(torch.bfloat16)
        d = [aclnn.from_torch(t) for t in (x, words, scale, offset, out)]
        ws_bytes = aclnn.weight_quant_batch_matmul(d[0], d[1], d[2], d[4], d[3], None, 128)
        workspace = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        call = lambda i: aclnn.weight_quant_batch_matmul(d[0], d[1], d[2], d[4], d[3], None, 128, workspace=workspace)  # noqa: E731
        nbytes = k * n // 2 + 2 * (k // 128) * n * 2 + 2 * m * k + 2 * m * n
    elif kind.startswith("int8_kc"):
        tb = kind.endswith("_t")
        x1 = torch.randint(-127, 128, (m, k), generator=gen, device=dev, dtype=torch.int8)
        x2s = [torch.randint(-127, 128, (n, k) if tb else (k, n), generator=gen, device=dev, dtype=torch.int8) for _ in range(sets)]
        s1 = torch.rand((m,), generator=gen, device=dev) * 9e-3 + 1e-3
        s2 = torch.rand((n,), generator=gen, device=dev) * 9e-3 + 1e-3
        bias = torch.randint(-1000, 1001, (n,), generator=gen, device=dev, dtype=torch.int32)
        d = [aclnn.from_torch(t) for t in (x1, s1, s2, bias)]
        dx2 = [aclnn.from_torch(t) for t in x2s]
        dout = aclnn.from_torch(out)
        call = lambda i: aclnn.quant_matmul_v5(d[0], dx2[i % sets], d[1], d[2], dout, d[3], False, tb)  # noqa: E731
        nbytes = m * k + k * n + 4 * (m + 2 * n) + 2 * m * n
    else:
        tb = kind.endswith("_t")
        wshape = (n, k) if tb else (k, n)
        if kind.startswith("int8_perblock"):
            x1 = torch.randint(-127, 128, (m, k), generator=gen, device=dev, dtype=torch.int8)
            x2s = [torch.randint(-127, 128, wshape, generator=gen, device=dev, dtype=torch.int8) for _ in range(sets)]
        else:
            x1 = torch.randn((m, k), generator=gen, device=dev).to(torch.float8_e4m3fn)
            x2s = [torch.randn(wshape, generator=gen, device=dev).to(torch.float8_e4m3fn) for _ in range(sets)]
        s1 = torch.rand((m, k // 128), generator=gen, device=dev) + 0.5
        s2 = torch.rand((n // 128, k // 128) if tb else (k // 128, n // 128), generator=gen, device=dev) + 0.5
        d = [aclnn.from_torch(t) for t in (x1, s1, s2)]
        dx2 = [aclnn.from_torch(t) for t in x2s]
        dout = aclnn.from_torch(out)
        group = (1 << 32) | (128 << 16) | 128
        call = lambda i: aclnn.quant_matmul_v5(d[0], dx2[i % sets], d[1], d[2], dout, None, False, tb, group)  # noqa: E731
        nbytes = m * k + k * n + 4 * (m * k // 128 + k * n // 16384) + 2 * m * n
    for i in range(max(args.warmup, 3)):
        call(i)
    torch.cuda.synchronize()
    steps = args.steps
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    sampler = ClockSampler(0)
    sampler.start()
    torch.cuda._sleep(60_000_000)
    for i in range(steps):
        evs[i][0].record()
        call(i)
        evs[i][1].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ts = sorted(a.elapsed_time(b_) for a, b_ in evs)
    ms = sum(ts) / len(ts)
    flops = 2.0 * b * m * k * n
    tf = flops / (ms * 1e-3) / 1e12
    peak8 = 9000.0 if kind.startswith("mxfp4") else (2250.0 if kind == "w4a16_prefill" else 4500.0)
    print(json.dumps({"metric": "QBMM TFLOPS", "workload": args.workload, "kind": kind, "shape": [b, m, k, n], "value": tf,
                      "unit": "TOP/s" if kind.startswith("int8") else "TFLOP/s", "ms_per_step": ms, "ms_min": ts[0], "steps": steps,
                      "kernel": aclnn.last_kernel_name(), "frac_of_datasheet_dense_peak": tf / peak8, "datasheet_dense_peak": peak8,
                      "hbm_gbs_on_algorithmic_bytes": nbytes / (ms * 1e-3) / 1e9, "clocks": clocks, "weight_sets": sets}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sets", type=int, default=4, help="distinct weight sets rotated through (L2 defeat)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload in QMM_WORKLOADS:
        return run_qmm_workload(args)
    args.warmup = max(args.warmup, 3)

    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    aclnn = load_package().aclnn
    aclnn.lib()

    x, data = make_inputs(torch, dev, 1002 + rank, args.sets)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    d_x, d_y = aclnn.from_torch(x), aclnn.from_torch(y)
    descs = [(aclnn.from_torch(w), aclnn.from_torch(s), aclnn.from_torch(o)) for (w, s, o) in data]
    ws_bytes = aclnn.weight_quant_batch_matmul(d_x, descs[0][0], descs[0][1], d_y, descs[0][2], None, G)
    workspace = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    kernel_name = aclnn.last_kernel_name()

    def step(i):
        w, s, o = descs[i % len(descs)]
        aclnn.weight_quant_batch_matmul(d_x, w, s, d_y, o, None, G, workspace=workspace)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = aclnn.launch_count()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    # park the GPU on a ~30 ms spin so that every launch of the timed region is already queued when it starts:
    # the 20 us kernels are then timed back to back, not the Python loop that enqueues them
    torch.cuda._sleep(60_000_000)
    t_begin.record()
    for i in range(args.steps):
        evs[i][0].record()
        step(i)
        evs[i][1].record()
    t_end.record()
    barrier()
    launches = aclnn.launch_count() - launches0
    total_ms = t_begin.elapsed_time(t_end)
    per_launch_ms = sorted(a.elapsed_time(b) for a, b in evs)
    kernel_ms = sum(per_launch_ms) / len(per_launch_ms)

    # ---- the same workload in the API's high-performance precision mode (innerPrecise = 1), device resident ----
    def step_hp(i):
        w, s, o = descs[i % len(descs)]
        aclnn.weight_quant_batch_matmul(d_x, w, s, d_y, o, None, G, inner_precise=1, workspace=workspace)

    for i in range(args.warmup):
        step_hp(i)
    hp_kernel = aclnn.last_kernel_name()
    barrier()
    hp_evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda._sleep(60_000_000)
    for i in range(args.steps):
        hp_evs[i][0].record()
        step_hp(i)
        hp_evs[i][1].record()
    barrier()
    hp_ms = sorted(a.elapsed_time(b) for a, b in hp_evs)
    hp_kernel_ms = sum(hp_ms) / len(hp_ms)

    # ---- end to end from host buffers (x H2D + call + y D2H per step) ----
    hx = torch.empty((M, K), dtype=torch.bfloat16).pin_memory()
    hx.copy_(x.cpu())
    hy = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    hw = [t.cpu().pin_memory() for t in data[0]]
    barrier()
    tu0 = time.perf_counter()
    for dst, src in zip(data[0], hw):
        dst.copy_(src, non_blocking=True)
    torch.cuda.synchronize()
    weight_upload_ms = (time.perf_counter() - tu0) * 1e3
    e2e_steps = max(10, args.steps // 4)
    for i in range(3):
        x.copy_(hx, non_blocking=True)
        step(i)
        hy.copy_(y, non_blocking=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(e2e_steps):
        x.copy_(hx, non_blocking=True)
        step(i)
        hy.copy_(y, non_blocking=True)
    e1.record()
    barrier()
    e2e_serial_ms = e0.elapsed_time(e1) / e2e_steps

    # The same loop with the copies on their own streams (x of step i+1 goes up and y of step i-1 comes down while step i
    # computes; two buffers of each, ordered by events). Every step still copies its x from pinned host memory and its y
    # back, inside the timed region; the host enqueues in real time, nothing is parked.
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    xb = [x, torch.empty_like(x)]
    yb = [y, torch.empty_like(y)]
    hyb = [hy, torch.empty_like(hy).pin_memory()]
    dxb = [aclnn.from_torch(t) for t in xb]
    dyb = [aclnn.from_torch(t) for t in yb]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def pipelined(nsteps):
        for i in range(nsteps):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[b])  # the step that last read this x buffer
                xb[b].copy_(hx, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[b])
                s_cmp.wait_event(ev_out[b])  # the copy that last read this y buffer
                w, sc, of = descs[i % len(descs)]
                aclnn.weight_quant_batch_matmul(dxb[b], w, sc, dyb[b], of, None, G, workspace=workspace)
                ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                hyb[b].copy_(yb[b], non_blocking=True)
                ev_out[b].record(s_out)

    pipelined(4)
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(s_in)
    pipelined(e2e_steps)
    for st in (s_in, s_cmp):
        s_out.wait_stream(st)
    p1.record(s_out)
    barrier()
    e2e_pipe_ms = p0.elapsed_time(p1) / e2e_steps
    e2e_ms = min(e2e_serial_ms, e2e_pipe_ms)
    clocks = sampler.stop() if rank == 0 else None  # sampled from before the first timed launch to after the last timed copy

    if dist is not None:
        t = torch.tensor([total_ms, kernel_ms, e2e_ms, hp_kernel_ms, e2e_serial_ms, e2e_pipe_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, kernel_ms, e2e_ms, hp_kernel_ms, e2e_serial_ms, e2e_pipe_ms = [float(v) for v in t.tolist()]
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt.item())

    if rank == 0:
        ms_per_step = total_ms / args.steps
        value = world * ALGO_BYTES / (ms_per_step * 1e-3) / 1e9
        peak, peak_src = measured_peak()
        achieved = ALGO_BYTES / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": "W4A16 decode HBM GB/s (weight_quant_batch_matmul_v2, algorithmic bytes / time)",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded; shapes and value ranges of BASELINE config 2)",
            "config": {"workload": WORKLOAD_C2,
                       "sharding": "n-sharded, one [8192,28672] weight shard per GPU, x replicated, no collective",
                       "l2": "rotating %d weight sets (%d MB) > 126 MB L2" % (args.sets, args.sets * ALGO_BYTES // 1000000),
                       "kernel": kernel_name, "workspace_bytes": int(ws_bytes)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src, "algorithmic_bytes_per_launch": ALGO_BYTES,
                         "kernel_ms_avg": kernel_ms, "kernel_ms_min": per_launch_ms[0],
                         "frac_of_8TBps_datasheet": achieved / 8000.0},
            "e2e": {"value": world * ALGO_BYTES / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": M * K * 2,
                    "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_ms, "ms_per_step_one_stream": e2e_serial_ms,
                    "ms_per_step_copy_streams": e2e_pipe_ms, "weight_upload_ms": weight_upload_ms,
                    "note": "x copied from pinned host memory and y copied back every step (the faster of: everything on one stream; copies on their own streams, double buffered); the quantised weight is a static parameter uploaded once"},
            "gpu_launches": launches, "clocks": clocks,
            # not the contract line's mode: aclnnWeightQuantBatchMatmulV3 with innerPrecise = 1 (the reference's documented
            # high-performance mode for A16W4 per-group, m <= 16); per-launch CUDA events, same inputs and rotation
            "inner_precise_1": {"kernel": hp_kernel, "achieved": ALGO_BYTES / (hp_kernel_ms * 1e-3) / 1e9, "unit": "GB/s",
                                "frac": ALGO_BYTES / (hp_kernel_ms * 1e-3) / 1e9 / peak, "kernel_ms_avg": hp_kernel_ms,
                                "kernel_ms_min": hp_ms[0]},
        }
        traffic_file = os.path.join(ROOT, "profiles", "wqbmm_decode_c2_traffic.json")
        if os.path.exists(traffic_file):
            with open(traffic_file) as fh:
                line["roofline"]["traffic"] = json.load(fh).get("dram_bytes_per_launch")
        if not args.no_cpu_baseline and world == 1:
            xs = to_np_bf16(x)
            w0, s0, o0 = data[0]
            _, line["cpu_baseline"] = cpu_baseline_c2(xs, w0.cpu().numpy(), to_np_bf16(s0), to_np_bf16(o0))
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
