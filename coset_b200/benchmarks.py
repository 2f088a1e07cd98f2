"""Secondary benchmarks (the reference declares a `coset-benchmark` entry point that does not
exist, pyproject.toml:67).  One JSON line per measurement:

    python -m coset_b200.benchmarks qat        # E8HNLQLinear QAT step, W [3072, 768], 4096 bf16 tokens
    python -m coset_b200.benchmarks vlut       # code-domain matmul, W [4096, 4096], T in {1, 16, 256, 4096}
    python -m torch.distributed.run --nproc-per-node N -m coset_b200.benchmarks gradcomm
                                               # E8-quantised gradient exchange, BERT-base-shaped gradient
    python -m coset_b200.benchmarks profile-gemv | profile-gemv16 | profile-gemm | profile-gemm-pair
                                               # small fixed cases of the matmul kernels for a profiler capture

Timing: CUDA events on the current stream, warm-up first, inputs resident on the device.
Roofline denominators: MEASURED_PEAKS.json at the repository root when present, else the
fallbacks 6650 GB/s and 1590 TFLOP/s.
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def cuda_time(fn, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def graph_time(fn, calls=20, replays=10):
    """Device time per call with launch overhead removed: `calls` invocations captured into one CUDA
    graph, replayed `replays` times (the Python/ctypes call path costs tens of microseconds, more than
    the small-T kernels themselves)."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(calls):
            fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (calls * replays)


def graph_step_time(layer, x, t):
    """Forward + backward of the layer captured once into a CUDA graph and replayed (the layer's kernels
    only enqueue work on the current stream, so the whole step is capturable; the 1-in-256 statistics
    update is a host-side branch and is not part of the captured step)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            layer.zero_grad(set_to_none=True)
            ((layer(x) - t).float() ** 2).mean().backward()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    layer.zero_grad(set_to_none=True)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ((layer(x) - t).float() ** 2).mean().backward()
    return cuda_time(lambda: g.replay())


def iter_qat(cases=None):
    """Yields one record per (weights, tiling) case of the QAT step benchmark."""
    from .core.e8 import create_e8_hnlq_linear
    from .core.layers import e8_fake_quantize
    hbm, tf, src = peaks()
    torch.manual_seed(0)
    tokens, d_in, d_out = 4096, 768, 3072
    x = torch.randn(tokens, d_in, device="cuda").to(torch.bfloat16)
    t = torch.randn(tokens, d_out, device="cuda").to(torch.bfloat16)
    all_cases = [(tag, std, tiling)
                 for tag, std in (("literal std=0.02 (all weights quantise to 0)", 0.02), ("std=20 (55% non-zero weights)", 20.0))
                 for tiling in ("row", "block")]
    for tag, std, tiling in all_cases:
        if cases is not None and (std, tiling) not in cases:
            continue
        layer = create_e8_hnlq_linear(d_in, d_out, q=4, M=2, tiling=tiling, init_kwargs={"std": std}, device="cuda")

        def step():
            layer.zero_grad(set_to_none=True)
            y = layer(x)
            ((y - t).float() ** 2).mean().backward()

        ms = cuda_time(step)
        ms_graph = graph_step_time(layer, x, t)
        from .core.layers import GraphedTrainStep
        gstep = GraphedTrainStep(layer, lambda y, tt: ((y - tt).float() ** 2).mean(), (x, t))
        ms_gstep = cuda_time(lambda: gstep(x, t))
        beta = layer._beta().detach()
        bpt = layer.blocks_per_row if tiling == "row" else 1
        w = layer.weight.detach()
        fq = cuda_time(lambda: e8_fake_quantize(w, beta, bpt, 4, 2.0, torch.bfloat16))
        n_blocks = w.numel() // 8
        fq_bytes = n_blocks * (32 + 16 + 4) + beta.numel() * 4  # fp32 in, bf16 out, codes out, scales
        yield ({
            "bench": "qat_step", "weights": tag, "tiling": tiling, "tokens": tokens, "shape": [d_out, d_in],
            "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3),
            "graph_ms_per_step": ms_graph, "graph_tokens_per_s": tokens / (ms_graph * 1e-3),
            "graphed_train_step_ms": ms_gstep, "graphed_train_step_tokens_per_s": tokens / (ms_gstep * 1e-3),
            "note": "eager steps are bound by the Python / launch path; the graph replays the same forward + backward",
            "gemm_tflops_equiv": 3 * 2 * tokens * d_in * d_out / (ms * 1e-3) / 1e12,
            "fake_quant_fwd_ms": fq, "fake_quant_fwd_GBps": fq_bytes / (fq * 1e-3) / 1e9,
            "fake_quant_frac_of_hbm": fq_bytes / (fq * 1e-3) / 1e9 / hbm, "peaks": src})


def bench_qat():
    for rec in iter_qat():
        print(json.dumps(rec), flush=True)


def iter_vlut(tilings=("block", "row")):
    """Yields one record per (tiling, T, path) of the code-domain product benchmark."""
    from .vlut import E8CodeLinear
    hbm, tf, src = peaks()
    torch.manual_seed(0)
    n = 4096
    W = (torch.randn(n, n) * 0.02).cuda()
    for tiling, bpt, nbeta in (("block", 1, n * n // 8), ("row", n // 8, n)):
        if tiling not in tilings:
            continue
        beta = torch.full((nbeta,), 25.0, device="cuda")
        lin = E8CodeLinear.from_weight(W, beta, bpt, small_t_max=64)
        wbytes = n * n // 8 * 4 + nbeta * 4
        for T in (1, 16, 256, 4096):
            x = torch.randn(T, n, device="cuda").to(torch.bfloat16)
            lin(x)
            ms = graph_time(lambda: lin(x)) if T <= 256 else cuda_time(lambda: lin(x), iters=10)
            flops = 2.0 * T * n * n
            rec = {"bench": "vlut_matmul", "tiling": tiling, "T": T, "shape": [n, n], "ms": ms,
                   "tokens_per_s": T / (ms * 1e-3),
                   "path": ("E8CodeLinear default: code-domain kernel" if T <= 64 else
                            "E8CodeLinear default: cached dense bf16 copy + library GEMM" if T < lin.PAIR_GEMM_MIN_T else
                            "E8CodeLinear default: decode + tcgen05 cta_group::2 GEMM, bf16 result"),
                   "timing": "CUDA graph replay" if T <= 256 else "CUDA events over eager calls",
                   "peaks": src}
            if T <= 64:
                by = wbytes + T * n * 2 + T * n * 4
                rec.update({"bound": "hbm", "GBps": by / (ms * 1e-3) / 1e9, "frac": by / (ms * 1e-3) / 1e9 / hbm})
            else:
                rec.update({"bound": "tensor", "TFLOPs": flops / (ms * 1e-3) / 1e12, "frac": flops / (ms * 1e-3) / 1e12 / tf})
            yield rec
            if T >= lin.PAIR_GEMM_MIN_T:  # the library path beside it
                dense = lin._dense_bf16()
                msl = cuda_time(lambda: torch.nn.functional.linear(x, dense), iters=10)
                yield {"bench": "vlut_matmul", "tiling": tiling, "T": T, "shape": [n, n], "ms": msl, "tokens_per_s": T / (msl * 1e-3),
                       "path": "library GEMM on a cached dense bf16 copy (large_t_path='cublas')", "timing": "CUDA events over eager calls",
                       "bound": "tensor", "TFLOPs": flops / (msl * 1e-3) / 1e12, "frac": flops / (msl * 1e-3) / 1e12 / tf, "peaks": src}
            if T > 64:
                from .vlut import e8_dequant_gemm
                e8_dequant_gemm(lin.codes, lin.beta, bpt, x, None, check=True)
                ms2 = graph_time(lambda: e8_dequant_gemm(lin.codes, lin.beta, bpt, x, None), calls=10, replays=5)
                yield {"bench": "vlut_matmul", "tiling": tiling, "T": T, "shape": [n, n], "ms": ms2,
                       "tokens_per_s": T / (ms2 * 1e-3), "path": "fused tcgen05 dequant-GEMM (no dense weight in HBM)",
                       "timing": "CUDA graph replay", "bound": "tensor", "TFLOPs": flops / (ms2 * 1e-3) / 1e12,
                       "frac": flops / (ms2 * 1e-3) / 1e12 / tf, "peaks": src}
                from .vlut import e8_decode_gemm
                scratch = torch.empty(n * n, dtype=torch.bfloat16, device="cuda")
                e8_decode_gemm(lin.codes, lin.beta, bpt, x, None, check=True, scratch=scratch)
                ms3 = graph_time(lambda: e8_decode_gemm(lin.codes, lin.beta, bpt, x, None, scratch=scratch), calls=10, replays=5)
                yield {"bench": "vlut_matmul", "tiling": tiling, "T": T, "shape": [n, n], "ms": ms3,
                       "tokens_per_s": T / (ms3 * 1e-3),
                       "path": "decode to a transient bf16 buffer + TMA-fed tcgen05 cta_group::2 GEMM (two launches, no dense weight kept)",
                       "timing": "CUDA graph replay", "bound": "tensor", "TFLOPs": flops / (ms3 * 1e-3) / 1e12,
                       "frac": flops / (ms3 * 1e-3) / 1e12 / tf, "peaks": src}
                del scratch


def bench_vlut():
    for rec in iter_vlut():
        print(json.dumps(rec), flush=True)


def bench_d4():
    """D4 weight path clamp(projection(W beta) / beta) and Babai rounding on 2^26 blocks of 4."""
    from . import _lib
    from .core.babai import babai_project
    from .core.d4 import D4Lattice
    from .core.e8 import E8Lattice
    hbm, _, src = peaks()
    n = 1 << 26
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(n, 4, device="cuda", generator=g) * 0.02
    beta = torch.full((n,), 25.0, device="cuda")
    out = torch.empty_like(x)
    L = _lib.lib()

    def run():
        rc = L.coset_d4_quantize(_lib.ptr(x), 0, _lib.ptr(beta), _lib.SCALE_MUL_TILE, n, 1, 2.0, _lib.ptr(out), 0, _lib.stream())
        assert rc == 0

    ms = cuda_time(run, iters=20)
    by = n * 36
    print(json.dumps({"bench": "d4_quantize", "blocks": n, "ms": ms, "GBps": by / (ms * 1e-3) / 1e9,
                      "frac_of_hbm": by / (ms * 1e-3) / 1e9 / hbm, "bytes_per_block": 36, "peaks": src}), flush=True)
    for name, lat, nb in (("d4", D4Lattice(device="cuda"), n), ("e8", E8Lattice(device="cuda"), n // 2)):
        xb = x.view(nb, lat.d)
        ms = cuda_time(lambda: babai_project(xb, lat, 0.25), iters=20)
        by = nb * lat.d * 8
        print(json.dumps({"bench": f"babai_{name}", "blocks": nb, "ms": ms, "GBps": by / (ms * 1e-3) / 1e9,
                          "frac_of_hbm": by / (ms * 1e-3) / 1e9 / hbm, "note": "includes the output allocation of the Python call",
                          "peaks": src}), flush=True)


def bench_vlut_sharded():
    """Config-4 weight split along the output features over the ranks of a torchrun launch: every
    rank multiplies its [4096 / W, 4096] slice, one all-gather of the outputs follows."""
    import torch.distributed as dist
    from .vlut import ColumnParallelE8CodeLinear
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.manual_seed(0)
    n = 4096
    W = (torch.randn(n, n) * 0.02).cuda()
    beta = torch.full((n * n // 8,), 25.0, device="cuda")
    lin = ColumnParallelE8CodeLinear.from_weight(W, beta, 1, small_t_max=64)
    lin_peer = ColumnParallelE8CodeLinear.from_weight(W, beta, 1, small_t_max=64, transport="peer")
    for T in (1, 16, 256, 4096):
        x = torch.randn(T, n, device="cuda").to(torch.bfloat16)
        res = {}
        cases = [("sharded_ms", lambda: lin(x)), ("local_product_ms", lambda: lin.local(x))]
        if T <= 64:
            cases.insert(1, ("sharded_peer_stores_ms", lambda: lin_peer(x)))
        for name, fn in cases:
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                fn()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / 20], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[name] = float(t.item())
        if rank == 0:
            res.update({"bench": "vlut_matmul_column_parallel", "n_gpus": world, "T": T, "shape": [n, n],
                        "tokens_per_s": T / (res["sharded_ms"] * 1e-3), "gathered_bytes_per_rank": T * n // world * 4,
                        "timing": "CUDA events over eager calls, max over ranks"})
            print(json.dumps(res), flush=True)
    dist.destroy_process_group()


def bench_gradcomm():
    import torch.distributed as dist
    from .gradcomm import E8GradientExchange, bert_base_gradient_numel
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    n = bert_base_gradient_numel()
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    grad = torch.randn(n, device="cuda", generator=g) * 1e-3
    ex = E8GradientExchange(scale=500.0)
    ex_peer = E8GradientExchange(scale=500.0, transport="peer")
    out = torch.empty_like(grad)

    def quantised():
        ex.all_reduce_mean(grad, out=out)

    def quantised_peer():
        ex_peer.all_reduce_mean(grad, out=out)

    ref = grad.clone()

    def plain():
        ref.copy_(grad)
        if world > 1:
            dist.all_reduce(ref)
        ref.div_(world)

    res = {}
    cases = [("e8_exchange_ms", quantised), ("fp32_allreduce_ms", plain)]
    if world > 1:
        cases.insert(1, ("e8_exchange_peer_memory_ms", quantised_peer))
    for name, fn in cases:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 10], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = float(t.item())
    if rank == 0:
        hbm, _, src = peaks()
        n_blocks = n // 8
        hbm_bytes = n_blocks * 36 + world * n_blocks * 4 + n_blocks * 32
        res.update({"bench": "gradient_exchange", "n_gpus": world, "values": n, "scale": 500.0,
                    "wire_bytes_sent_per_rank": n_blocks * 4, "wire_bytes_fp32_ring_per_rank": 2 * (world - 1) / max(world, 1) * n * 4,
                    "gradient_GBps_per_gpu": n * 4 / (res["e8_exchange_ms"] * 1e-3) / 1e9,
                    "kernel_hbm_bytes": hbm_bytes, "hbm_floor_ms": hbm_bytes / (hbm * 1e9) * 1e3, "peaks": src,
                    "speedup_vs_fp32_allreduce": res["fp32_allreduce_ms"] / res["e8_exchange_ms"]})
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


def profile_case(which):
    """Small fixed cases for a profiler capture (W 4096 x 4096, per-block scales, bf16 tokens):
    `profile-gemv` / `profile-gemv16` run the few-token code-domain product five times at T = 1 / 16, `profile-gemm` the
    fused tcgen05 dequant-GEMM three times at T = 2048 and checks its status word, `profile-gemm-pair` the same with
    the decode + cta_group::2 GEMM."""
    from .vlut import E8CodeLinear, e8_decode_gemm, e8_dequant_gemm
    torch.manual_seed(0)
    n = 4096
    W = (torch.randn(n, n) * 0.02).cuda()
    beta = torch.full((n * n // 8,), 25.0, device="cuda")
    lin = E8CodeLinear.from_weight(W, beta, 1)
    if which in ("profile-gemv", "profile-gemv16"):
        x = torch.randn(1 if which == "profile-gemv" else 16, n, device="cuda").to(torch.bfloat16)
        for _ in range(5):
            lin(x)
    else:
        x = torch.randn(2048, n, device="cuda").to(torch.bfloat16)
        gemm = e8_decode_gemm if which == "profile-gemm-pair" else e8_dequant_gemm
        for _ in range(3):
            gemm(lin.codes, lin.beta, 1, x, None, check=True)
    torch.cuda.synchronize()
    print("ok")


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    which = argv[0] if argv else "all"
    if which in ("profile-gemv", "profile-gemv16", "profile-gemm", "profile-gemm-pair"):
        profile_case(which)
        return
    if which in ("qat", "all"):
        bench_qat()
    if which in ("vlut", "all"):
        bench_vlut()
    if which in ("d4", "all"):
        bench_d4()
    if which == "vlut_sharded":
        bench_vlut_sharded()
    if which in ("gradcomm", "all"):
        bench_gradcomm()


if __name__ == "__main__":
    main()
