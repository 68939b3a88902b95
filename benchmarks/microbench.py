"""Micro-benchmarks of the native kernels against the measured device peaks.

``python -m benchmarks.microbench [gemm|norm|ce|adam|attn|small|all]`` (from the repository
root) times each
kernel with CUDA events (3 warm-up launches, L2 flushed between timed launches by
writing a 256 MB buffer) and prints achieved TFLOP/s or GB/s, plus the same
shape through torch (cuBLAS / eager) for comparison.
"""
from __future__ import annotations

import json
import sys

import torch


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(flush):
    from necklace_b200.ops import gemm
    shapes = [  # (M, N, K, a_mn, b_mn, label)
        (8192, 3072, 1024, False, False, "qkv fwd"),
        (8192, 1024, 1024, False, False, "proj fwd"),
        (8192, 4096, 1024, False, False, "fc1 fwd"),
        (8192, 1024, 4096, False, False, "fc2 fwd"),
        (8192, 1024, 4096, False, True, "fc1 dgrad"),
        (4096, 1024, 8192, True, True, "fc1 wgrad"),
        (8192, 50304, 1024, False, False, "lm head"),
        (8192, 8192, 8192, False, False, "square 8k"),
    ]
    rows = []
    for M, N, K, a_mn, b_mn, label in shapes:
        A = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        B = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda: gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out), flush=flush)
        At = A.t() if a_mn else A
        Bt = B if b_mn else B.t()
        ms_t = _time(lambda: torch.matmul(At, Bt, out=out), flush=flush)
        fl = 2.0 * M * N * K
        ms_1 = _time(lambda: gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, bn=256), flush=flush)
        ms_2 = _time(lambda: gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, bn=512), flush=flush)
        rows.append({"op": "gemm", "label": label, "M": M, "N": N, "K": K, "ms": round(ms, 4),
                     "tflops": round(fl / ms / 1e9, 1),
                     "tflops_1cta_256": round(fl / ms_1 / 1e9, 1),
                     "tflops_pair_256x256": round(fl / ms_2 / 1e9, 1),
                     "torch_ms": round(ms_t, 4), "torch_tflops": round(fl / ms_t / 1e9, 1)})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def bench_norm(flush):
    from necklace_b200.ops.norm import norm_fwd, norm_bwd
    rows, C = 65536, 1024
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w = torch.ones(C, device="cuda").bfloat16()
    b = torch.zeros(C, device="cuda").bfloat16()
    ms = _time(lambda: norm_fwd(x, w, b, 1e-5, False), flush=flush)
    y, st = norm_fwd(x, w, b, 1e-5, False)
    ms_b = _time(lambda: norm_bwd(x, x, w, st, False), flush=flush)
    byts = rows * C * 2
    print(json.dumps({"op": "layernorm_fwd", "ms": round(ms, 4), "GBps": round(2 * byts / ms / 1e6)}))
    print(json.dumps({"op": "layernorm_bwd(dx+dw+db)", "ms": round(ms_b, 4),
                      "GBps_min_traffic": round(3 * byts / ms_b / 1e6)}), flush=True)


def bench_colsum(flush):
    from necklace_b200.ops.gemm import colsum
    for (rows, C) in [(8192, 1024), (8192, 3072), (8192, 4096)]:
        dy = torch.randn(rows, C, device="cuda").bfloat16()
        out = torch.empty(C, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda: colsum(dy, out), flush=flush)
        print(json.dumps({"op": "colsum", "rows": rows, "C": C, "ms": round(ms, 4),
                          "GBps": round(rows * C * 2 / ms / 1e6)}), flush=True)


def bench_ce(flush):
    from necklace_b200.ops import cross_entropy_fwd_bwd
    T, V, ld = 8192, 50257, 50304
    lg = torch.randn(T, ld, device="cuda").bfloat16()
    tg = torch.randint(0, V, (T,), device="cuda")
    ms = _time(lambda: cross_entropy_fwd_bwd(lg, tg, V, 1.0 / T), flush=flush)
    print(json.dumps({"op": "ce_fwd_bwd", "ms": round(ms, 4),
                      "GBps": round(2 * T * ld * 2 / ms / 1e6)}), flush=True)


def bench_adam(flush):
    from necklace_b200.ops import adam_step
    n = 355_000_000
    master = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    g = torch.randn(n, device="cuda").bfloat16()
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: adam_step(master, m, v, g, pb, lr=1e-4, step=2), iters=5)
    print(json.dumps({"op": "adam_flat", "n": n, "ms": round(ms, 4),
                      "GBps": round(n * (12 * 2 + 2 + 2) / ms / 1e6)}), flush=True)


def bench_attn(flush):
    from necklace_b200.ops.attention import attn_fwd, attn_bwd
    for (B, H, S, D) in [(8, 16, 1024, 64), (2, 32, 2048, 128), (1, 40, 4096, 128)]:
        C = H * D
        qkv = torch.randn(B, S, 3 * C, device="cuda").bfloat16()
        from necklace_b200.ops.attention import set_exp_mode, set_fwd_impl
        q_, k_, v_ = (t.view(B, S, H, D).transpose(1, 2).float() for t in qkv.split(C, -1))
        ref = torch.nn.functional.scaled_dot_product_attention(q_, k_, v_, is_causal=True)
        ref = ref.transpose(1, 2).reshape(B, S, C)
        modes = {}
        for impl, mode in ((0, 0), (0, 1), (1, 1), (1, 0)):
            set_fwd_impl(impl)
            set_exp_mode(mode)
            t_ms = _time(lambda: attn_fwd(qkv, H, True), flush=flush)
            o_, _ = attn_fwd(qkv, H, True)
            err = ((o_.float() - ref).norm() / ref.norm()).item()
            modes[f"impl{impl}_exp{mode}"] = {"ms": round(t_ms, 4), "rel_err": round(err, 5)}
        print(json.dumps({"op": "attn_fwd_exp_modes", "B": B, "H": H, "S": S, "D": D, **modes}),
              flush=True)
        ms = _time(lambda: attn_fwd(qkv, H, True), flush=flush)
        out, lse = attn_fwd(qkv, H, True)
        do = torch.randn_like(out)
        ms_b = _time(lambda: attn_bwd(qkv, out, lse, do, H, True), flush=flush)
        from necklace_b200.ops.attention import set_bwd_impl
        set_bwd_impl(0)
        ms_b0 = _time(lambda: attn_bwd(qkv, out, lse, do, H, True), flush=flush)
        set_bwd_impl(1)
        fl = 4.0 * B * H * S * S * D / 2  # causal
        q, k, v = (t.view(B, S, H, D).transpose(1, 2) for t in qkv.split(C, -1))
        ms_t = _time(lambda: torch.nn.functional.scaled_dot_product_attention(
            q, k, v, is_causal=True), flush=flush)
        print(json.dumps({"op": "attn", "B": B, "H": H, "S": S, "D": D, "fwd_ms": round(ms, 4),
                          "fwd_tflops": round(fl / ms / 1e9, 1), "bwd_ms": round(ms_b, 4),
                          "bwd_serial_ms": round(ms_b0, 4),
                          "bwd_tflops": round(2.5 * fl / ms_b / 1e9, 1),
                          "torch_sdpa_fwd_ms": round(ms_t, 4)}), flush=True)


def bench_small(flush):
    """``small``: three launches each (one warm-up, two timed) of the memory-bound kernels and of the 3x3 convolution
    (im2col gather + tcgen05 GEMM, forward and both gradients) on cases a few hundred MB in
    size: larger than L2, small enough for a counter capture of single launches."""
    from necklace_b200.ops import adam_step, cross_entropy_fwd_bwd
    from necklace_b200.ops.conv import Conv2d
    from necklace_b200.ops.norm import norm_bwd, norm_fwd
    rows, C = 65536, 1024
    x = torch.randn(rows, C, device="cuda").bfloat16()
    w = torch.ones(C, device="cuda").bfloat16()
    b = torch.zeros(C, device="cuda").bfloat16()
    y, st = norm_fwd(x, w, b, 1e-5, False)
    ms = _time(lambda: norm_fwd(x, w, b, 1e-5, False), iters=2, warmup=1, flush=flush)
    ms_b = _time(lambda: norm_bwd(x, x, w, st, False), iters=2, warmup=1, flush=flush)
    byts = rows * C * 2
    print(json.dumps({"op": "layernorm_fwd", "rows": rows, "C": C, "ms": round(ms, 4),
                      "GBps": round(2 * byts / ms / 1e6)}))
    print(json.dumps({"op": "layernorm_bwd", "ms": round(ms_b, 4),
                      "GBps_min_traffic": round(3 * byts / ms_b / 1e6)}), flush=True)
    T, V, ld = 2048, 50257, 50304
    lg = torch.randn(T, ld, device="cuda").bfloat16()
    tg = torch.randint(0, V, (T,), device="cuda")
    ms = _time(lambda: cross_entropy_fwd_bwd(lg, tg, V, 1.0 / T), iters=2, warmup=1, flush=flush)
    print(json.dumps({"op": "ce_fwd_bwd", "T": T, "V": V, "ms": round(ms, 4),
                      "GBps": round(2 * T * ld * 2 / ms / 1e6)}), flush=True)
    n = 32 * 1024 * 1024
    master = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    g = torch.randn(n, device="cuda").bfloat16()
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: adam_step(master, m, v, g, pb, lr=1e-4, step=2), iters=2, warmup=1,
               flush=flush)
    print(json.dumps({"op": "adam_flat", "n": n, "ms": round(ms, 4),
                      "GBps": round(n * (12 * 2 + 2 + 2) / ms / 1e6)}), flush=True)
    del master, m, v, g, pb, lg
    N, H, Cc = 256, 56, 64
    conv = Conv2d(Cc, Cc, k=3, stride=1, pad=1, device="cuda")
    xi = torch.randn(N, H, H, Cc, device="cuda").bfloat16().requires_grad_(True)
    dy = torch.randn(N, H, H, Cc, device="cuda").bfloat16()

    def fb():
        xi.grad = None
        conv.weight.grad = None
        conv(xi).backward(dy)
    ms = _time(fb, iters=2, warmup=1, flush=flush)
    fl = 3 * 2.0 * N * H * H * Cc * Cc * 9
    print(json.dumps({"op": "conv3x3 fwd+bwd", "N": N, "HW": H, "C": Cc, "ms": round(ms, 4),
                      "tflops": round(fl / ms / 1e9, 1)}), flush=True)


def one_gemm(argv):
    """``gemm_one M N K [a_mn b_mn [epilogue]]``: a handful of launches of one shape (ncu
    captures); epilogue: none | bias | gelu (bias + GELU, saves the pre-activation) |
    gelubwd (times GELU' of a saved pre-activation) | res (bias + residual)."""
    from necklace_b200.ops import gemm, EPI_GELU_FWD, EPI_GELU_BWD
    M, N, K = (int(x) for x in argv[2:5])
    a_mn = len(argv) > 5 and argv[5] == "1"
    b_mn = len(argv) > 6 and argv[6] == "1"
    epi = argv[7] if len(argv) > 7 else "none"
    A = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    B = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda").bfloat16()
    aux = torch.randn(M, N, device="cuda").bfloat16()
    kw = {}
    if epi == "bias":
        kw = dict(bias=bias)
    elif epi == "gelu":
        kw = dict(bias=bias, epi=EPI_GELU_FWD, aux=aux)
    elif epi == "gelubwd":
        kw = dict(epi=EPI_GELU_BWD, aux=aux)
    elif epi == "res":
        kw = dict(bias=bias, res=aux)
    for _ in range(5):
        gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, **kw)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(20):
        gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, **kw)
    ev[1].record()
    torch.cuda.synchronize()
    print(json.dumps({"op": "gemm_one", "M": M, "N": N, "K": K, "epi": epi,
                      "ms": round(ev[0].elapsed_time(ev[1]) / 20, 4)}), flush=True)


def one_attn(argv):
    """``attn_one B H S D``: a few forward+backward launches of one shape (ncu captures)."""
    from necklace_b200.ops.attention import attn_fwd, attn_bwd
    B, H, S, D = (int(x) for x in argv[2:6])
    qkv = torch.randn(B, S, 3 * H * D, device="cuda").bfloat16()
    for _ in range(3):
        out, lse = attn_fwd(qkv, H, True)
        attn_bwd(qkv, out, lse, out, H, True)
    torch.cuda.synchronize()


def main(argv):
    which = argv[1] if len(argv) > 1 else "all"
    if which == "gemm_one":
        return one_gemm(argv)
    if which == "attn_one":
        return one_attn(argv)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    table = {"gemm": bench_gemm, "colsum": bench_colsum, "norm": bench_norm, "ce": bench_ce, "adam": bench_adam,
             "attn": bench_attn}
    if which == "small":
        bench_small(flush)
    for name, fn in table.items():
        if which in ("all", name):
            fn(flush)
    from necklace_b200.ops import check_status
    check_status()


if __name__ == "__main__":
    main(sys.argv)
