#!/usr/bin/env python
"""Headline benchmark: bulk E8 HNLQ codec throughput (encode + decode GB/s, fraction of HBM peak).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config "bulk codec"): float32 [2^25, 8] (2^28 values), N(0, 0.02) with 0.1 %
of the entries replaced by +-10 sigma outliers, clipped to +-2, q=4, M=2, one float32 scale per
8-value block in the layer (multiply) convention.  One STEP = one encode pass (x -> packed
codes) followed by one decode pass (codes -> x_hat) over the whole batch.  Algorithmic bytes per
block: encode 32 + 4 + 4, decode 4 + 4 + 32 => 80 B per block per step.

The literal scale of that config (beta at theta=0 = 0.02144) maps every block to the all-zero
code, so the headline uses beta = 25 (scaled sigma 0.5: every branch of the search is exercised,
about half the blocks take the parity flip and ~45 % the half-integer coset); the literal scale
is reported next to it under "detail".

Multi-GPU (--gpus N under torch.distributed.run): blocks are independent, each rank runs the
same per-GPU workload on its own seed (weak scaling, no data-path collective); the time is the
max over ranks.
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_BLOCKS = 1 << 25
BYTES_PER_BLOCK_ENC = 40
BYTES_PER_BLOCK_DEC = 40
BYTES_PER_BLOCK_STEP = BYTES_PER_BLOCK_ENC + BYTES_PER_BLOCK_DEC
BETA_HEADLINE = 25.0
BETA_LITERAL = 0.021440971642732620
FALLBACK_HBM_GBS = 6650.0


def encode_traffic_bytes(n_blocks):
    """DRAM read + write bytes of one encode launch over n_blocks blocks: the counters of one profiler
    capture of the same kernel on a smaller case (kept as data next to its summary), scaled by the
    number of blocks.  None when no capture is on record."""
    p = os.path.join(ROOT, "profiles", "codec_q4m2_bulk_fp32.json")
    try:
        d = json.load(open(p))
        return (float(d["dram_bytes_read"]) + float(d["dram_bytes_write"])) * n_blocks / float(d["capture_blocks"])
    except Exception:
        return None


def make_values(n_values, seed):
    """The config's synthetic distribution, generated in fixed chunks of 2^24 values."""
    g = torch.Generator().manual_seed(seed)
    out = torch.empty(n_values, dtype=torch.float32)
    chunk = 1 << 24
    for lo in range(0, n_values, chunk):
        n = min(chunk, n_values - lo)
        v = torch.randn(n, generator=g) * 0.02
        m = torch.rand(n, generator=g) < 1e-3
        s = torch.randint(0, 2, (n,), generator=g) * 2 - 1
        v[m] = 0.2 * s[m].float()
        out[lo:lo + n] = v.clamp_(-2.0, 2.0)
    return out


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) from a thread while the
    timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index, period_s=0.002):
        import threading
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._mark = 0
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it is a plain list
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[index]) if index < len(ids) else index
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        for bit, name in self.REASONS.items():
                            if mask & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception as e:  # NVML missing: the line then carries "clocks": null
            self.error = repr(e)

    def mark(self):
        """Start of the timed steps: samples before this belong to the warm-up (same load)."""
        self._mark = len(self.samples)

    def stop(self):
        if self._thread is None:
            return None
        self._stop.set()
        self._thread.join(timeout=2)
        if not self.samples:
            return None
        timed = self.samples[self._mark:]
        # an NVML query takes milliseconds; when the timed steps are shorter than three queries the
        # warm-up steps (the same kernels on the same data, back to back) are included and named
        window = "timed steps" if len(timed) >= 3 else "warm-up + timed steps (same load, back to back)"
        self.samples = timed if len(timed) >= 3 else self.samples
        self.window = window
        return {"window": window, "sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def time_kernels(fn_list, steps, warmup):
    """Runs the kernels of one step in order, `steps` times; returns (total ms, per-kernel mean ms)."""
    for _ in range(warmup):
        for fn in fn_list:
            fn()
    torch.cuda.synchronize()
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(fn_list) + 1)] for _ in range(steps)]
    for s in range(steps):
        marks[s][0].record()
        for i, fn in enumerate(fn_list):
            fn()
            marks[s][i + 1].record()
    torch.cuda.synchronize()
    total = marks[0][0].elapsed_time(marks[-1][-1])
    per = [sum(m[i].elapsed_time(m[i + 1]) for m in marks) / steps for i in range(len(fn_list))]
    return total, per


def cpu_port_throughput(x_cpu, beta_cpu, sample_blocks, threads, repeats=1):
    """The CPU oracle (C restatement of the reference) on a prefix of the workload, all host cores."""
    from oracle import oracle as O
    xs = x_cpu[:sample_blocks].numpy()
    bs = beta_cpu[:sample_blocks].numpy()
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        codes = O.encode(xs, beta=bs, scale_mode=2, blocks_per_tile=1, q=4, M=2, threads=threads)
        O.decode(codes, beta=bs, scale_mode=2, blocks_per_tile=1, q=4, threads=threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_blocks * BYTES_PER_BLOCK_STEP / best / 1e9, best


def parity_check(x_cpu, beta_cpu, codes, xhat, sample=1 << 16):
    """The codes and reconstructions the timed kernels left in their output buffers, compared bit for
    bit with the CPU oracle on the first `sample` blocks (outside the timed region)."""
    import numpy as np
    from oracle import oracle as O
    k = min(sample, x_cpu.shape[0])
    digits = O.encode(x_cpu[:k].numpy(), beta=beta_cpu[:k].numpy(), scale_mode=2, blocks_per_tile=1, threads=os.cpu_count() or 1)
    want_x = O.decode(digits, beta=beta_cpu[:k].numpy(), scale_mode=2, blocks_per_tile=1, threads=os.cpu_count() or 1)
    got_c = codes[:k].view(torch.int32).view(-1).cpu().numpy().view(np.uint32)
    got_x = xhat[:k].cpu().numpy()
    return {"sample_blocks": k, "codes_bit_exact": bool(np.array_equal(got_c, O.pack_q4(digits))),
            "reconstruction_bit_exact": bool(np.array_equal(got_x.view(np.uint32), (want_x + np.float32(0)).view(np.uint32))),
            "against": "CPU oracle (C restatement of coset.core.e8)"}


def gradient_exchange_detail(rank, world, iters=10):
    """E8-quantised gradient exchange on the BERT-base-shaped gradient (109 482 240 values, N(0, 1e-3),
    seed 1000 + rank, scale 500), per transport: time (CUDA events, max over ranks), the phases of the
    all-gather form, the plain float32 all-reduce beside it, and a bit-for-bit check of rank 0's result
    against the CPU recipe on every 64th block."""
    import numpy as np
    import torch.distributed as dist
    from coset_b200.gradcomm import E8GradientExchange, bert_base_gradient_numel
    n_values = bert_base_gradient_numel()
    n_blocks = n_values // 8
    scale = 500.0
    g = torch.Generator().manual_seed(1000 + rank)
    grad = (torch.randn(n_values, generator=g) * 1e-3).cuda()
    out = torch.empty_like(grad)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # the CPU recipe on every 64th block needs every rank's sample of the input
    sample = grad.view(n_blocks, 8)[::64].contiguous()
    samples = torch.empty((world,) + tuple(sample.shape), dtype=torch.float32, device="cuda")
    dist.all_gather_into_tensor(samples.view(-1), sample.view(-1))
    want = None
    if rank == 0:
        from oracle import oracle as O
        total = None
        for r in range(world):
            # the exchange's encode: x * scale in float32, clamped to +-3.9 (saturating encode), then the codec
            xs = (samples[r].cpu().numpy() * np.float32(scale)).astype(np.float32)
            d = O.encode(np.clip(xs, np.float32(-3.9), np.float32(3.9)), threads=os.cpu_count() or 1)
            xh = O.decode(d)
            total = xh if total is None else (total + xh).astype(np.float32)
        want = (total / np.float32(np.float32(scale) * np.float32(world))).astype(np.float32)

    res = {"values": n_values, "scale": scale, "wire_bytes_sent_per_rank": n_blocks * 4,
           "wire_bytes_received_per_rank": (world - 1) * n_blocks * 4}
    ref = grad.clone()

    def plain():
        ref.copy_(grad)
        dist.all_reduce(ref)
        ref.div_(world)
    res["fp32_allreduce_ms"] = timed(plain)
    for transport in ("nccl", "peer"):
        ex = E8GradientExchange(scale=scale, transport=transport)
        ms = timed(lambda: ex.all_reduce_mean(grad, out=out))
        rec = {"ms": ms, "gradient_GBps_per_gpu": n_values * 4 / (ms * 1e-3) / 1e9,
               "nvlink_rx_GBps": (world - 1) * n_blocks * 4 / (ms * 1e-3) / 1e9,
               "frac_of_900GBps": (world - 1) * n_blocks * 4 / (ms * 1e-3) / 1e9 / 900.0,
               "speedup_vs_fp32_allreduce": res["fp32_allreduce_ms"] / ms}
        if transport == "nccl":  # phases: encode | all-gather | decode-and-average (events on this rank)
            ex.phase_events = []
            for _ in range(5):
                ex.all_reduce_mean(grad, out=out)
            torch.cuda.synchronize()
            ev, ph = ex.phase_events, [0.0, 0.0, 0.0]
            for i in range(0, len(ev), 4):
                for j in range(3):
                    ph[j] += ev[i + j].elapsed_time(ev[i + j + 1]) / (len(ev) // 4)
            ex.phase_events = None
            t = torch.tensor(ph, dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rec["phases_ms"] = dict(zip(("encode", "all_gather", "decode_mean"), [float(v) for v in t]))
            rec["bound_by"] = max(rec["phases_ms"], key=rec["phases_ms"].get)
        ex.all_reduce_mean(grad, out=out)
        torch.cuda.synchronize()
        if rank == 0:
            got = out.view(n_blocks, 8)[::64].cpu().numpy()
            rec["matches_cpu_recipe"] = bool(np.array_equal((got + np.float32(0)).view(np.uint32), (want + np.float32(0)).view(np.uint32)))
        res[transport] = rec
        del ex
    return res


def column_parallel_detail(rank, world, iters=20):
    """Code-domain product [4096, 4096] sharded along the output features over the ranks: per token
    count the time of the sharded layer (all-gather of the outputs, or peer stores for few tokens), the
    local product alone, and a bit-for-bit comparison with the unsharded layer on the same device."""
    import torch.distributed as dist
    from coset_b200.vlut import ColumnParallelE8CodeLinear, E8CodeLinear
    torch.manual_seed(0)
    n = 4096
    W = (torch.randn(n, n) * 0.02).cuda()
    beta = torch.full((n * n // 8,), 25.0, device="cuda")
    full = E8CodeLinear.from_weight(W, beta, 1)
    lin = ColumnParallelE8CodeLinear.from_weight(W, beta, 1)
    lin_peer = ColumnParallelE8CodeLinear.from_weight(W, beta, 1, transport="peer")
    out = {}
    for T in (1, 16, 256, 4096):
        x = torch.randn(T, n, device="cuda").to(torch.bfloat16)
        cases = [("all_gather_ms", lambda: lin(x)), ("local_product_ms", lambda: lin.local(x))]
        if T <= lin.local.small_t_max:
            cases.append(("peer_stores_ms", lambda: lin_peer(x)))
        rec = {}
        for name, fn in cases:
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / iters], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rec[name] = float(t.item())
        same = torch.equal(lin(x), full(x))
        if T <= lin.local.small_t_max:
            same = same and torch.equal(lin_peer(x), full(x))
        flag = torch.tensor([1 if same else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        rec["matches_unsharded"] = bool(int(flag.item()))
        rec["tokens_per_s"] = T / (min(v for k, v in rec.items() if k in ("all_gather_ms", "peer_stores_ms")) * 1e-3)
        rec["gathered_bytes_per_rank"] = T * n // world * 4
        out[f"T={T}"] = rec
    return out


def base_line(args, world):
    return {
        "metric": "E8 HNLQ encode+decode GB/s (% HBM peak)",
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic (seeded N(0,0.02) + 0.1% +-10sigma outliers, clip 2.0)",
        "config": {
            "workload": "bulk E8 HNLQ codec: fp32 [2^25, 8] per GPU, q=4, M=2, per-block scale beta=25 "
                        "(layer/multiply convention); step = encode pass + decode pass, 80 B/block",
            "n_blocks_per_gpu": N_BLOCKS,
            "q": 4, "M": 2, "beta": BETA_HEADLINE,
            "l2": "inputs (1 GiB per pass) larger than L2, no flush needed",
        },
    }


def run_reference(args, rank, world):
    """The reference's CPU path (C port of coset.core.e8, all host threads) on a bounded sample."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = 1 << 21
    x = make_values(sample * 8, 0).view(sample, 8)
    beta = torch.full((sample,), BETA_HEADLINE)
    for _ in range(args.warmup):
        cpu_port_throughput(x, beta, sample, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_port_throughput(x, beta, sample, threads)
    dt = time.perf_counter() - t0
    value = args.steps * sample * BYTES_PER_BLOCK_STEP / dt / 1e9
    line = base_line(args, world)
    line.update({
        "impl": "reference", "value": value, "ms_per_step": dt / args.steps * 1e3, "gpu_launches": 0,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"first {sample} blocks of the workload per step (1/16 of a GPU step)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--blocks", type=int, default=N_BLOCKS, help="blocks per GPU (default: the config's 2^25)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-detail", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-comm", action="store_true", help="skip the gradient-exchange / column-parallel section of a multi-GPU run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    from coset_b200 import _lib
    from coset_b200.core.e8 import e8_decode_packed, e8_encode_packed
    from coset_b200.core.e8.codecs import _lib as _  # noqa: F401  (fails loudly if the CUDA library is missing)

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    n = args.blocks
    x_cpu = make_values(n * 8, rank).view(n, 8)
    beta_cpu = torch.full((n,), BETA_HEADLINE)
    x = x_cpu.cuda()
    beta = beta_cpu.cuda()
    codes = torch.empty((n, 4), dtype=torch.uint8, device="cuda")
    xhat = torch.empty((n, 8), dtype=torch.float32, device="cuda")
    MT = _lib.SCALE_MUL_TILE

    def enc():
        e8_encode_packed(x, 4, 2, scale=beta, scale_mode=MT, blocks_per_tile=1, out=codes)

    def dec():
        e8_decode_packed(codes, 4, 2, scale=beta, scale_mode=MT, blocks_per_tile=1, out=xhat)

    # ---- timed region: K steps of (encode, decode), inputs resident in HBM
    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(args.warmup):
        enc(); dec()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark()
    total_ms, per = time_kernels([enc, dec], args.steps, 0)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    value = world * args.steps * n * BYTES_PER_BLOCK_STEP / (total_ms * 1e-3) / 1e9

    # ---- end to end through the host-buffer API (pinned host arrays in, host arrays out)
    e2e = None
    if not args.no_e2e:
        from coset_b200.host import HostCodec
        hc = HostCodec(chunk_blocks=1 << 21, n_slots=4)
        xh = x_cpu.pin_memory()
        bh = beta_cpu.pin_memory()
        ch = torch.empty((n, 4), dtype=torch.uint8, pin_memory=True)
        oh = torch.empty((n, 8), dtype=torch.float32, pin_memory=True)
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            hc.encode(xh, scale=bh, scale_mode=MT, out=ch); hc.decode(ch, scale=bh, scale_mode=MT, out=oh)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            hc.encode(xh, scale=bh, scale_mode=MT, out=ch)
            hc.decode(ch, scale=bh, scale_mode=MT, out=oh)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": world * e2e_steps * n * BYTES_PER_BLOCK_STEP / float(dt.item()) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": n * (32 + 4 + 4 + 4), "d2h_bytes_per_step": n * (4 + 32), "steps": e2e_steps,
               "api": "coset_b200.host.HostCodec.encode/.decode -> coset_e8_encode_host / coset_e8_decode_host"}
        ok = torch.equal(oh[:4096], xhat[:4096].cpu())
        e2e["matches_device_path"] = bool(ok)
        # the same host arrays through the one-pass round trip (codes and reconstruction both returned;
        # the codes are not uploaded again, so both PCIe directions are busy at once)
        oh2 = torch.empty((n, 8), dtype=torch.float32, pin_memory=True)
        hc.quantize(xh, scale=bh, scale_mode=MT, out=oh2, codes_out=ch)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            hc.quantize(xh, scale=bh, scale_mode=MT, out=oh2, codes_out=ch)
        torch.cuda.synchronize()
        dt2 = time.perf_counter() - t0
        e2e["one_pass_roundtrip"] = {"value": e2e_steps * n * BYTES_PER_BLOCK_STEP / dt2 / 1e9, "unit": "GB/s (this rank)",
                                     "h2d_bytes_per_step": n * (32 + 4), "d2h_bytes_per_step": n * (32 + 4),
                                     "api": "HostCodec.quantize -> coset_e8_quantize_host",
                                     "matches_two_call_path": bool(torch.equal(oh2[:4096], oh[:4096]))}
        del oh2
        hc.close()
        del xh, ch, oh

    # ---- detail: each kernel alone, the fused round trip, bf16, and the literal (degenerate) scale
    detail = {}
    if not args.no_detail and rank == 0:
        from coset_b200 import _lib as L
        k = max(5, min(args.steps, 20))

        def gbs(ms, bytes_per_block):
            return n * bytes_per_block / (ms * 1e-3) / 1e9

        _, p = time_kernels([enc], k, 3); detail["encode_f32_GBps"] = gbs(p[0], 40)
        _, p = time_kernels([dec], k, 3); detail["decode_f32_GBps"] = gbs(p[0], 40)
        out = torch.empty_like(x)

        def rt():
            rc = L.lib().coset_e8_quantize(L.ptr(x), 0, L.ptr(beta), MT, n, 1, 4, 2, 0.0, L.ptr(out), 0, None, L.stream())
            L.check(rc, "coset_e8_quantize")
        _, p = time_kernels([rt], k, 3); detail["roundtrip_f32_GBps"] = gbs(p[0], 68)
        del out
        xb = x.to(torch.bfloat16)
        ob = torch.empty_like(xb)

        def encb():
            e8_encode_packed(xb, 4, 2, scale=beta, scale_mode=MT, blocks_per_tile=1, out=codes)

        def decb():
            e8_decode_packed(codes, 4, 2, scale=beta, scale_mode=MT, blocks_per_tile=1, out=ob)
        _, p = time_kernels([encb, decb], k, 3)
        detail["encode_bf16_GBps"] = gbs(p[0], 24); detail["decode_bf16_GBps"] = gbs(p[1], 24)
        del xb, ob
        beta_lit = torch.full((n,), BETA_LITERAL, device="cuda")

        def encl():
            e8_encode_packed(x, 4, 2, scale=beta_lit, scale_mode=MT, blocks_per_tile=1, out=codes)

        def decl():
            e8_decode_packed(codes, 4, 2, scale=beta_lit, scale_mode=MT, blocks_per_tile=1, out=xhat)
        tl, p = time_kernels([encl, decl], k, 3)
        detail["literal_beta_theta0"] = {"beta": BETA_LITERAL, "encode_GBps": gbs(p[0], 40), "decode_GBps": gbs(p[1], 40),
                                         "encode+decode_GBps": gbs(p[0] + p[1], 80), "note": "all codes are zero at this scale"}
        enc(); dec()  # restore headline buffers
        if world == 1:
            # the other two workloads of the metric (quantized-linear tokens/s), one GPU
            from coset_b200 import benchmarks as B
            keep = ("tiling", "ms_per_step", "tokens_per_s", "graph_ms_per_step", "graph_tokens_per_s", "graphed_train_step_ms",
                    "graphed_train_step_tokens_per_s", "fake_quant_fwd_ms", "fake_quant_frac_of_hbm")
            detail["qat"] = {("literal_std0.02" if r["weights"].startswith("literal") else "std20"): {k: r[k] for k in keep}
                             for r in B.iter_qat(cases=((0.02, "row"), (20.0, "row")))}
            detail["qat"]["workload"] = ("E8HNLQLinear QAT step: W [3072, 768], 4096 bf16 tokens, forward + backward; ms_per_step = eager, "
                                         "graph_* = the step replayed as one CUDA graph, graphed_train_step_* = the public "
                                         "GraphedTrainStep helper (input copies and the layer's host-side bookkeeping included)")
            detail["vlut"] = [{k: r[k] for k in ("T", "ms", "tokens_per_s", "path", "timing", "bound", "frac") if k in r} |
                              ({"TFLOPs": r["TFLOPs"]} if "TFLOPs" in r else {"GBps": r["GBps"]})
                              for r in B.iter_vlut(tilings=("block",))]

    # ---- parity of what the timed kernels produced (rank 0, sample vs the CPU oracle)
    parity = parity_check(x_cpu, beta_cpu, codes, xhat) if rank == 0 and not args.no_cpu else None

    # ---- the paths that communicate (multi-GPU runs only; every rank takes part)
    comm = None
    if world > 1 and not args.no_comm:
        del x, xhat, codes
        torch.cuda.empty_cache()
        comm = {"gradcomm": gradient_exchange_detail(rank, world), "vlut_column_parallel": column_parallel_detail(rank, world)}

    # ---- CPU baseline (rank 0, single-GPU run only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        sample = min(n, 1 << 22)
        v, secs = cpu_port_throughput(x_cpu, beta_cpu, sample, threads)
        cpu = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"first {sample} of {n} blocks, one encode+decode pass, {secs:.2f} s"}

    if rank == 0:
        peak, peak_src = hbm_peak()
        enc_ms = per[0]
        achieved = n * BYTES_PER_BLOCK_ENC / (enc_ms * 1e-3) / 1e9
        line = base_line(args, world)
        line["config"]["n_blocks_per_gpu"] = n
        line.update({
            "value": value,
            "ms_per_step": total_ms / args.steps,
            "gpu_launches": 3 * args.steps,  # per step: k_encode_q4m2_main, k_encode_q4m2_fix, k_decode_q4m2
            "frac_of_hbm_peak": value / world / peak,
            "roofline": {"bound": "hbm", "kernel": "encode pass = k_encode_q4m2_main + its fix-up launch k_encode_q4m2_fix (dominant: %.0f%% of the step)" % (100 * per[0] / (per[0] + per[1])),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": encode_traffic_bytes(n), "algorithmic_bytes_per_launch": n * BYTES_PER_BLOCK_ENC,
                         "peak_source": peak_src, "ms_per_launch": enc_ms,
                         "decode": {"achieved": n * BYTES_PER_BLOCK_DEC / (per[1] * 1e-3) / 1e9, "ms_per_launch": per[1]}},
            "clocks": clocks,
            "e2e": e2e,
            "cpu_baseline": cpu,
            "parity": parity,
            "detail": detail,
        })
        if comm is not None:
            line["detail"].update(comm)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
