#!/usr/bin/env python
"""Operator-level benchmarks of the hand-written kernels against the library baselines on the same box.

  python bench_ops.py --only gemm,flash,bw,mamba            (one GPU)
  torchrun --nproc-per-node N ... bench_ops.py --only tp    (fused tensor-parallel kernels against NCCL + GEMM)

Timing: CUDA events on the launching stream after warm-up, an L2 flush (256 MB write) between timed iterations, median
of the iterations; multi-GPU numbers are the max over ranks.  Prints one JSON line per measurement and writes them to
--out when given.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oa_b200.ops import kernels as K  # noqa: E402

RESULTS = []


def emit(**kw):
    RESULTS.append(kw)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(kw), flush=True)


def timeit(fn, iters=15, warm=4, flush=True):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    ts = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm():
    shapes = [(16384, 4096, 1024, 0, 0), (16384, 1024, 4096, 0, 0), (16384, 3072, 1024, 0, 0), (16384, 1024, 1024, 0, 0),
              (8192, 8192, 8192, 0, 0), (16384, 1024, 4096, 0, 1), (4096, 1024, 16384, 1, 1), (16384, 32000, 1024, 0, 0)]
    for (M, N, Kk, amn, bmn) in shapes:
        a = torch.randn((Kk, M) if amn else (M, Kk), device="cuda").bfloat16()
        b = torch.randn((Kk, N) if bmn else (N, Kk), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda: K.gemm(a, b, a_mn=bool(amn), b_mn=bool(bmn), out=out))
        A, B = (a.t() if amn else a), (b if bmn else b.t())
        t2 = timeit(lambda: torch.matmul(A, B, out=out))
        fl = 2 * M * N * Kk
        emit(op="gemm_bf16", M=M, N=N, K=Kk, a_mn=amn, b_mn=bmn, ms=t, tflops=fl / t / 1e9, cublas_ms=t2, cublas_tflops=fl / t2 / 1e9)
    K.check_status()


def bench_gemm_epilogue():
    """The fused epilogues of the flagship's FFN GEMMs against the plain product of the same shape (the epilogue should hide
    under the next tile's main loop) and against the library sequence that a framework without fusion runs."""
    import torch.nn.functional as Fn
    M, D, Ff = 16384, 1024, 4096
    x = torch.randn(M, D, device="cuda").bfloat16()
    w1 = torch.randn(Ff, D, device="cuda").bfloat16() * 0.03
    g = torch.randn(M, D, device="cuda").bfloat16()
    w2 = torch.randn(D, Ff, device="cuda").bfloat16() * 0.03
    z = torch.empty(M, Ff, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(M, Ff, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, D, device="cuda").bfloat16()
    o = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    t_plain = timeit(lambda: K.gemm(x, w1, out=h))
    t_gelu = timeit(lambda: K.gemm(x, w1, act=K.ACT_GELU, aux_out=z, out=h))
    t_bwd = timeit(lambda: K.gemm(g, w2, b_mn=True, act=K.ACT_GELU_BWD, aux_in=z, out=h))
    t_bwd_plain = timeit(lambda: K.gemm(g, w2, b_mn=True, out=h))
    t_res = timeit(lambda: K.gemm(h, w2, residual=res, out=o))
    t_res_plain = timeit(lambda: K.gemm(h, w2, out=o))

    def lib_fwd():
        torch.matmul(x, w1.t(), out=z)
        return Fn.gelu(z, approximate="tanh")

    t_lib = timeit(lib_fwd)
    emit(op="gemm_epilogue", M=M, N=Ff, K=D, plain_ms=t_plain, gelu_aux_out_ms=t_gelu, gelu_bwd_aux_in_ms=t_bwd, gelu_bwd_plain_ms=t_bwd_plain,
         residual_ms=t_res, residual_plain_ms=t_res_plain, cublas_plus_gelu_kernel_ms=t_lib)
    K.check_status()


def bench_gemm_small_m():
    """Weight-streaming GEMMs of a decode step (32 rows): time against weight bytes, own kernel and cuBLAS."""
    for (M, N, Kk) in [(32, 12288, 4096), (32, 4096, 4096), (32, 22016, 4096), (32, 4096, 11008), (32, 32000, 4096)]:
        a = torch.randn(M, Kk, device="cuda").bfloat16()
        b = torch.randn(N, Kk, device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda: K.gemm(a, b, out=out))
        t2 = timeit(lambda: torch.matmul(a, b.t(), out=out))
        emit(op="gemm_bf16_small_m", M=M, N=N, K=Kk, us=t * 1e3, weight_gbs=N * Kk * 2 / t / 1e6, cublas_us=t2 * 1e3,
             cublas_weight_gbs=N * Kk * 2 / t2 / 1e6)
    K.check_status()


def bench_flash():
    import torch.nn.functional as Fn
    for (B, H, S, hd) in [(8, 16, 2048, 64), (1, 32, 4096, 128)]:
        D = H * hd
        qkv = torch.randn(B * S, 3 * D, device="cuda").bfloat16()
        q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
        t = timeit(lambda: K.flash_fwd(q, k, v, B, S, H, hd, causal=True))
        o, lse = K.flash_fwd(q, k, v, B, S, H, hd, causal=True)
        do = torch.randn_like(o)
        dqkv = torch.empty_like(qkv)
        tb = timeit(lambda: K.flash_bwd(q, k, v, o, do, lse, B, S, H, hd, causal=True, dqkv=dqkv))
        mk = lambda t_: t_.reshape(B, S, H, hd).transpose(1, 2).contiguous().requires_grad_(True)
        q4, k4, v4 = mk(q), mk(k), mk(v)
        ts = timeit(lambda: Fn.scaled_dot_product_attention(q4, k4, v4, is_causal=True))
        oo = Fn.scaled_dot_product_attention(q4, k4, v4, is_causal=True)
        g = torch.randn_like(oo)
        tsb = timeit(lambda: torch.autograd.grad(oo, (q4, k4, v4), g, retain_graph=True))
        fl = 4 * B * H * S * S * hd / 2
        emit(op="flash_attention_causal", B=B, H=H, S=S, hd=hd, fwd_ms=t, fwd_tflops=fl / t / 1e9, bwd_ms=tb, bwd_tflops=2.5 * fl / tb / 1e9,
             sdpa_fwd_ms=ts, sdpa_bwd_ms=tsb)
    K.check_status()


def bench_bw():
    x = torch.randn(16384, 1024, device="cuda").bfloat16()
    w = torch.randn(1024, device="cuda").bfloat16()
    t = timeit(lambda: K.rmsnorm_fwd(x, w, 1e-5))
    emit(op="rmsnorm_fwd", rows=16384, cols=1024, us=t * 1e3, gbs=2 * x.numel() * 2 / t / 1e6)
    _, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
    t = timeit(lambda: K.rmsnorm_bwd(x, w, x, rstd))
    emit(op="rmsnorm_bwd", rows=16384, cols=1024, us=t * 1e3, gbs=3 * x.numel() * 2 / t / 1e6)
    t = timeit(lambda: K.rmsnorm_bwd(x, w, x, rstd, dres=x))
    emit(op="rmsnorm_bwd_with_residual_gradient", rows=16384, cols=1024, us=t * 1e3, gbs=4 * x.numel() * 2 / t / 1e6)
    qkv = torch.randn(16384, 3072, device="cuda").bfloat16()
    t = timeit(lambda: K.rope_(qkv[:, :2048], 32, 64, 2048))          # q and k of a packed projection, in place
    emit(op="rope_inplace_packed_qk", rows=16384, heads=32, head_dim=64, us=t * 1e3, gbs=2 * 16384 * 2048 * 2 / t / 1e6)
    lg = torch.randn(16384, 32000, device="cuda").bfloat16()
    tg = torch.randint(0, 32000, (16384,), device="cuda")
    t = timeit(lambda: K.xent_fwd_bwd(lg, tg, grad_scale=1.0, dlogits=lg))
    emit(op="xent_fwd_bwd_inplace", rows=16384, vocab=32000, us=t * 1e3, gbs=2 * lg.numel() * 2 / t / 1e6)
    n = 335_000_000
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    g = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ms, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    st = torch.tensor([1, 1e-3, 0.9, 0.999, 1e-8, 0.1, 1.0, 0], device="cuda")
    t = timeit(lambda: K.adam_step(p, g, ms, m, v, st, decoupled=True))
    emit(op="adamw_step", n=n, ms=t, gbs=n * 28 / t / 1e6)


def bench_image():
    """Image kernels on a batch of 8 RGB 1080p frames (199 MB, larger than L2): algorithmic bytes = one read + one write."""
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.vision import fn_detection as D
    from oa_b200.vision import fn_image as I
    x = OaMatrix(torch.rand(8, 3, 1080, 1920, device="cuda"))
    nbytes = x.Tensor().numel() * 4
    k7 = OaMatrix(torch.rand(7, 7, device="cuda"))
    cases = {"brightness_contrast": lambda: I.BrightnessContrast(x, 0.1, 1.2), "gaussian_blur_sigma2 (13 taps, separable)": lambda: I.GaussianBlur(x, 2.0),
             "convolve2d_7x7": lambda: I.Convolve2d(x, k7), "erode_5x5": lambda: I.Erode(x, 5, 5), "median_5x5": lambda: I.MedianBlur(x, 5),
             "bilateral_5x5": lambda: I.BilateralFilter(x, 5), "flip": lambda: I.Flip(x, True, False)}
    for name, fn in cases.items():
        t = timeit(fn, iters=9, warm=3)
        emit(op="image." + name, shape=[8, 3, 1080, 1920], ms=t, gbs=2 * nbytes / t / 1e6)
    t = timeit(lambda: I.Resize(x, 960, 540), iters=9, warm=3)
    emit(op="image.resize_bilinear_half", shape=[8, 3, 1080, 1920], ms=t, gbs=1.25 * nbytes / t / 1e6)
    n = 20000
    boxes = torch.cat([torch.rand(n, 2, device="cuda") * 1000, torch.rand(n, 2, device="cuda") * 60 + 4], 1)
    scores = torch.rand(n, device="cuda")
    classes = torch.randint(0, 80, (n,), device="cuda", dtype=torch.int32)
    t = timeit(lambda: D.Nms(OaMatrix(boxes), OaMatrix(scores), OaMatrix(classes), D.OaNmsConfig(MaxDetections=300)), iters=9, warm=3, flush=False)
    emit(op="detection.nms", boxes=n, classes=80, max_detections=300, ms=t)
    K.check_status()


def bench_mamba():
    from oa_b200.ops import mamba3 as M3
    for (B, L, H, P, Nn) in [(4, 4096, 48, 64, 128), (2, 1024, 48, 64, 128)]:
        d = M3.Mamba3Dims(d_inner=H * P, heads=H, headdim=P, d_state=Nn, angles=32, has_z=True, chunk=256)
        proj = (torch.randn(B * L, d.d_in_proj, device="cuda") * 0.5).bfloat16()
        dtb = torch.rand(1, H, device="cuda")
        Bb, Cb, D = torch.ones(H, Nn, device="cuda"), torch.ones(H, Nn, device="cuda"), torch.zeros(H, device="cuda")
        tf = timeit(lambda: M3.core_fwd(proj, dtb, Bb, Cb, D, d, B, L, save=True), iters=5, warm=2)
        y, saved = M3.core_fwd(proj, dtb, Bb, Cb, D, d, B, L, save=True)
        dy = torch.randn_like(y)
        tb = timeit(lambda: M3.core_bwd(saved, dy), iters=5, warm=2)
        emit(op="mamba3_core", B=B, L=L, H=H, P=P, N=Nn, fwd_ms=tf, bwd_ms=tb, tokens_per_s_fwd_bwd=B * L / ((tf + tb) / 1e3))
    K.check_status()


def bench_mamba_once():
    """One forward + backward of the Mamba-3 core at B=2, L=4096 (no timing loop): the workload of the per-launch profile."""
    from oa_b200.ops import mamba3 as M3
    B, L, H, P, Nn = 2, 4096, 48, 64, 128
    d = M3.Mamba3Dims(d_inner=H * P, heads=H, headdim=P, d_state=Nn, angles=32, has_z=True, chunk=256)
    proj = (torch.randn(B * L, d.d_in_proj, device="cuda") * 0.5).bfloat16()
    dtb = torch.rand(1, H, device="cuda")
    Bb, Cb, D = torch.ones(H, Nn, device="cuda"), torch.ones(H, Nn, device="cuda"), torch.zeros(H, device="cuda")
    for _ in range(2):
        y, saved = M3.core_fwd(proj, dtb, Bb, Cb, D, d, B, L, save=True)
        M3.core_bwd(saved, torch.randn_like(y))
    torch.cuda.synchronize()
    K.check_status()
    emit(op="mamba3_core_once", B=B, L=L, status="ok")


def bench_decode_attn():
    """Single-query attention over the KV cache of one layer of the 7B-class decode case: streamed kernel against the
    one-CTA-per-head kernel (bytes = K and V rows read once)."""
    B, H, S, L, hd = 32, 32, 2304, 2200, 128
    kc = torch.randn(B, H, S, hd, device="cuda").bfloat16()
    vc = torch.randn(B, H, S, hd, device="cuda").bfloat16()
    q = torch.randn(B, H * hd, device="cuda").bfloat16()
    nbytes = 2 * B * H * L * hd * 2
    for name in ("stream", "v1"):
        os.environ["OA_DECODE_ATTN"] = name
        t = timeit(lambda: K.decode_attn(q, kc, vc, L), iters=15, warm=4)
        emit(op="decode_attn." + name, batch=B, heads=H, length=L, head_dim=hd, us=t * 1e3, gbs=nbytes / t / 1e6)
    os.environ.pop("OA_DECODE_ATTN", None)
    K.check_status()


def bench_decode():
    """Batch-32 greedy decoding of 256 tokens after a 2048-token prompt on the 7B-class model (one GPU, KV cache)."""
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.types import OaPrecision
    from oa_b200.models import OaGptConfig, OaGptModel
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    from oa_b200.serve import OaGptDecoder
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=0))
    F.SetRngSeed(1)
    cfg = OaGptConfig.Llama7B()
    model = OaGptModel(cfg)
    B, S, NEW = 32, 2048, 256
    prompt = torch.randint(0, cfg.Vocab, (B, S), dtype=torch.int32, device="cuda")
    dec = OaGptDecoder(model, batch=B, max_seq=S + NEW)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    dec.Prefill(prompt[:, :256])                 # warm-up of every kernel shape family
    dec.Step(prompt[:, :1])
    torch.cuda.synchronize()
    e[0].record()
    logits = dec.Prefill(prompt)
    e[1].record()
    for _ in range(NEW):
        nxt = logits.float().argmax(-1).to(torch.int32).reshape(-1, 1)
        logits = dec.Step(nxt)
    e[2].record()
    torch.cuda.synchronize()
    t_pre, t_dec = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
    emit(op="decode_7b_kv_cache", batch=B, prompt=S, new_tokens=NEW, prefill_ms=t_pre, prefill_tokens_per_s=B * S / t_pre * 1e3,
         decode_ms_per_token=t_dec / NEW, decode_tokens_per_s=B * NEW / t_dec * 1e3, kv_cache_gb=dec.Cache.Bytes() / 1e9,
         weight_gb=sum(p.NumElements() for p in model.AllParameterPtrs()) * 2 / 1e9)
    K.check_status()


def bench_prof():
    """A small fixed workload for profiler captures: every hot kernel twice (operands larger than L2, about 1 GB held)."""
    a = torch.randn(8192, 4096, device="cuda").bfloat16()
    b = torch.randn(4096, 4096, device="cuda").bfloat16()
    out = torch.empty(8192, 4096, device="cuda", dtype=torch.bfloat16)
    B, H, S, hd = 8, 16, 2048, 64
    D = H * hd
    qkv = torch.randn(B * S, 3 * D, device="cuda").bfloat16()
    q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
    x = torch.randn(65536, 1024, device="cuda").bfloat16()
    w = torch.randn(1024, device="cuda").bfloat16()
    lg = torch.randn(4096, 32000, device="cuda").bfloat16()
    tg = torch.randint(0, 32000, (4096,), device="cuda")
    n = 64_000_000
    p_ = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    g_ = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ms, m, vv = (torch.zeros(n, device="cuda") for _ in range(3))
    st = torch.tensor([1, 1e-3, 0.9, 0.999, 1e-8, 0.1, 1.0, 0], device="cuda")
    for _ in range(2):
        K.gemm(a, b, out=out)
        o, lse = K.flash_fwd(q, k, v, B, S, H, hd, causal=True)
        K.flash_bwd(q, k, v, o, o, lse, B, S, H, hd, causal=True, dqkv=torch.empty_like(qkv))
        _, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
        K.rmsnorm_bwd(x, w, x, rstd)
        K.xent_fwd_bwd(lg, tg, grad_scale=1.0, dlogits=lg)
        K.adam_step(p_, g_, ms, m, vv, st, decoupled=True)
    torch.cuda.synchronize()
    K.check_status()
    emit(op="prof_workload", done=True)


def bench_tp():
    import torch.distributed as dist
    from oa_b200.parallel import tp as TP
    from oa_b200.parallel.mesh import OaDeviceMesh
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mesh = OaDeviceMesh()
    arena = TP.OaTpArena(mesh, 1 << 30)
    M, D, Fd = 4096, 4096, 11008
    Fl = (Fd // world + 7) // 8 * 8

    def maxr(t):
        x = torch.tensor([t], device="cuda", dtype=torch.float64)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x)

    def loop(fn, n=10):
        def run():
            for _ in range(n):
                fn()
        return timeit(run, iters=7, warm=2, flush=False) / n

    for name, Kd, Nn in (("qkv", D, 3 * D // world), ("gate_up", D, 2 * Fl)):
        site = TP.OaTpAgSite(arena, M, Kd)
        xs = torch.randn(M // world, Kd, device="cuda").bfloat16()
        w = (torch.randn(Nn, Kd, device="cuda") * 0.02).bfloat16()
        full = torch.empty(M, Kd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, Nn, device="cuda", dtype=torch.bfloat16)
        t = maxr(loop(lambda: TP.ag_gemm(site, xs, w)))
        emit(op="tp_allgather_gemm_fused", site=name, world=world, M=M, N=Nn, K=Kd, us=t * 1e3, tflops=2 * M * Nn * Kd / t / 1e9)

        def base():
            dist.all_gather_into_tensor(full, xs)
            K.gemm(full, w, out=out)

        def base_cublas():
            dist.all_gather_into_tensor(full, xs)
            torch.matmul(full, w.t(), out=out)

        t1, t2 = maxr(loop(base)), maxr(loop(base_cublas))
        tg = maxr(loop(lambda: K.gemm(full, w, out=out)))
        emit(op="tp_allgather_gemm_baseline", site=name, world=world, M=M, N=Nn, K=Kd, nccl_plus_own_gemm_us=t1 * 1e3,
             nccl_plus_cublas_us=t2 * 1e3, gemm_only_us=tg * 1e3, nvlink_bytes=(world - 1) * (M // world) * Kd * 2)
    for name, Kd in (("attn_out", D // world), ("ffn_down", Fl)):
        site = TP.OaTpRsSite(arena, M, D)
        a = torch.randn(M, Kd, device="cuda").bfloat16()
        w = (torch.randn(D, Kd, device="cuda") * 0.02).bfloat16()
        res = torch.randn(M // world, D, device="cuda").bfloat16()
        part = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
        outs = torch.empty(M // world, D, device="cuda", dtype=torch.bfloat16)
        t = maxr(loop(lambda: TP.gemm_rs(site, a, w, residual=res)))
        emit(op="tp_gemm_reducescatter_fused", site=name, world=world, M=M, N=D, K=Kd, us=t * 1e3, tflops=2 * M * D * Kd / t / 1e9)

        def base():
            K.gemm(a, w, out=part)
            dist.reduce_scatter_tensor(outs, part)
            K.binary("add", outs, res, out=outs)

        def base_cublas():
            torch.matmul(a, w.t(), out=part)
            dist.reduce_scatter_tensor(outs, part)
            outs.add_(res)

        t1, t2 = maxr(loop(base)), maxr(loop(base_cublas))
        emit(op="tp_gemm_reducescatter_baseline", site=name, world=world, M=M, N=D, K=Kd, own_gemm_plus_nccl_us=t1 * 1e3,
             cublas_plus_nccl_us=t2 * 1e3, nvlink_bytes=(world - 1) * (M // world) * D * 2)
    torch.cuda.synchronize()
    K.check_status()
    mesh.Close()
    dist.destroy_process_group()


def bench_misc():
    """LunarLander3d stepping (lanes per second), row compaction / scatter / accuracy counters / stochastic rounding and the
    resize backward kernel, each on inputs larger than L2; algorithmic bytes as stated per case."""
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.ops import lunar as LL
    from oa_b200.vision import fn_image as I
    p = LL.LunarParams()
    terrain = LL.make_terrain(p, 1).cuda()
    E = 1 << 18
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device="cuda")
    sf, su, tr, obs = z(E, 32), z(E, 16, dt=torch.int32), z(E, 33), z(E, 33)
    rew, term, trunc, reason, stop = z(E), z(E, dt=torch.uint8), z(E, dt=torch.uint8), z(E, dt=torch.int32), z(E, dt=torch.uint8)
    LL.reset(p, terrain, sf, su, obs, 7, False)
    action = torch.randint(0, 8, (E,), device="cuda", dtype=torch.int32)

    def step():
        LL.step(p, terrain, action, stop, sf, su, tr, obs, rew, term, trunc, reason)
        LL.reset(p, terrain, sf, su, obs, 7, True)
    t = timeit(step, iters=9, warm=3)
    emit(op="rl.lunar_lander3d_step+reset", lanes=E, ms=t, lanes_per_s=E / t * 1e3, gbs=E * (2 * 192 + 2 * 132 + 4 + 10) / t / 1e6)
    T, D = 1 << 20, 64
    x = OaMatrix(torch.randn(T, D, device="cuda", dtype=torch.bfloat16))
    mask = OaMatrix((torch.rand(T, device="cuda") > 0.5).float())
    r = F.CompactRows(x, mask)
    nb = T * D * 2
    t = timeit(lambda: F.CompactRows(x, mask), iters=9, warm=3)
    emit(op="rows.compact", shape=[T, D], dtype="bf16", ms=t, gbs=(nb + nb / 2 + nb) / t / 1e6)             # read x, write half, zero-fill
    base = OaMatrix(torch.zeros(T, D, device="cuda", dtype=torch.bfloat16))
    t = timeit(lambda: F.ScatterRows(base, r.Values, r), iters=9, warm=3)
    emit(op="rows.scatter", shape=[T, D], dtype="bf16", ms=t, gbs=(2 * nb + nb) / t / 1e6)                  # clone base, move half in and out
    logits = OaMatrix(torch.randn(1 << 15, 8192, device="cuda", dtype=torch.bfloat16))
    labels = OaMatrix(torch.randint(0, 8192, (1 << 15,), device="cuda", dtype=torch.int32))
    t = timeit(lambda: F.CategoricalAccuracyCount(logits, labels), iters=9, warm=3)
    emit(op="accuracy_count", shape=[1 << 15, 8192], dtype="bf16", ms=t, gbs=(1 << 15) * 8192 * 2 / t / 1e6)
    w = OaMatrix(torch.randn(1 << 27, device="cuda"))
    t = timeit(lambda: F.SrRoundBf16(w, 3), iters=9, warm=3)
    emit(op="sr_round_bf16", n=1 << 27, ms=t, gbs=(1 << 27) * 6 / t / 1e6)
    g = OaMatrix(torch.rand(8, 3, 540, 960, device="cuda"))
    t = timeit(lambda: I.ResizeBilinearBwd(g, 1080, 1920), iters=9, warm=3)
    emit(op="image.resize_bilinear_bwd_2x", shape=[8, 3, 1080, 1920], ms=t, gbs=(8 * 3 * 540 * 960 * 4 + 8 * 3 * 1080 * 1920 * 4) / t / 1e6)
    K.check_status()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="gemm,flash,bw")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    table = {"gemm": bench_gemm, "flash": bench_flash, "bw": bench_bw, "mamba": bench_mamba, "mamba1": bench_mamba_once, "tp": bench_tp, "decode": bench_decode, "prof": bench_prof, "image": bench_image, "decode_attn": bench_decode_attn, "gemm_small_m": bench_gemm_small_m, "gemm_epi": bench_gemm_epilogue, "misc": bench_misc}
    for name in args.only.split(","):
        table[name.strip()]()
    if args.out and int(os.environ.get("RANK", "0")) == 0:
        with open(args.out, "w") as f:
            json.dump(RESULTS, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
