"""Per-kernel device timing at the headline shapes, with roofline fractions.

``python -m cosmos_predict25_b200.ops.bench_kernels [--quick] [--only NAME] [--json PATH]``

Each row: kernel, shape, CUDA-event time (median of timed iterations after warm-up, L2 flushed between
iterations by writing a 256 MB buffer), achieved TFLOP/s or GB/s, and the fraction of the measured
peak (``MEASURED_PEAKS.json`` at the repository root when present, otherwise 6.65 TB/s and
1.59 PFLOP/s). The library twin (cuBLAS / cuDNN via torch) is timed next to each contraction.

``--reference`` adds the reference arm of the attention rows: the reference repository's own, unmodified
``cosmos_predict2/_src/predict2/networks/attention.py`` (its dispatcher) and
``cosmos_predict2/_src/predict2/utils/flash_attention_jvp_triton.py`` (its Triton forward-mode kernel) are loaded by file
path from ``baseline/_ref`` (a copy of the reference tree) and timed on the same tensors.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys

import torch

from . import functional as F_ops
from . import native


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "src": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, iters=5, warmup=3):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush_l2()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def _load_reference_module(rel_path: str, name: str):
    """Import one file of the reference tree under ``baseline/_ref`` as a stand-alone module (None when it is absent)."""
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "baseline", "_ref", rel_path)
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", action="store_true", help="also time the reference repository's own attention code (baseline/_ref)")
    ap.add_argument("--quick", action="store_true", help="1/8 of the tokens (fast sanity pass)")
    ap.add_argument("--only", default=None)
    ap.add_argument("--json", default=None)
    ap.add_argument("--variants", action="store_true", help="also time the tuning variants of kernels that have them")
    ap.add_argument("--seq", type=int, default=None, help="override the token count (small cases for profiler captures)")
    ap.add_argument("--heads", type=int, default=None, help="override the head count of the attention rows")
    ap.add_argument("--no-twin", action="store_true", help="skip the library twins")
    args = ap.parse_args()
    ops = native.load()
    pk = peaks()
    N = args.seq or (84480 // (8 if args.quick else 1))
    D, H, HD, Fm, L, T = 2048, 16, 128, 8192, 3520 // (8 if args.quick else 1), 24
    rows = []

    def add(name, shape, ms, flops=None, bytes_=None, note=""):
        r = {"kernel": name, "shape": shape, "ms": round(ms, 4), "note": note}
        if flops is not None:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["frac_of_" + pk["src"] + "_bf16_peak"] = round(flops / ms / 1e9 / pk["tflops"], 3)
        if bytes_ is not None:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r["frac_of_" + pk["src"] + "_hbm"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)
        rows.append(r)
        print(json.dumps(r), flush=True)

    def want(name):
        return args.only is None or args.only in name

    torch.manual_seed(0)
    dev = "cuda"
    if want("gemm"):
        for (M, Nn, K, tag) in [(N, D, D, "qkv/out proj"), (N, Fm, D, "mlp.layer1"), (N, D, Fm, "mlp.layer2")]:
            a = torch.randn(M, K, device=dev).bfloat16()
            b = torch.randn(Nn, K, device=dev).bfloat16()
            fl = 2.0 * M * Nn * K
            add("gemm_tcgen05 nt", f"{M}x{Nn}x{K} {tag}", time_ms(lambda: ops.gemm_bf16(a, b, None, 0, False, False)), fl)
            prev = ops.gemm_pair_mode(1 - ops.gemm_pair_mode(-1))          # the other tile mode (CTA pairs <-> single CTA)
            add(f"gemm_tcgen05 nt, {'CTA pairs (256 x 256 per cluster)' if prev == 0 else 'single-CTA tiles'}", f"{M}x{Nn}x{K} {tag}",
                time_ms(lambda: ops.gemm_bf16(a, b, None, 0, False, False)), fl)
            ops.gemm_pair_mode(prev)
            add("cublas nt (twin)", f"{M}x{Nn}x{K}", time_ms(lambda: torch.matmul(a, b.T)), fl)
        a = torch.randn(N, D, device=dev).bfloat16()
        b = torch.randn(Fm, D, device=dev).bfloat16()
        add("gemm_tcgen05 nt +gelu(+pre)", f"{N}x{Fm}x{D}", time_ms(lambda: ops.gemm_bf16_gelu_pre(a, b, None)), 2.0 * N * Fm * D)
        dy = torch.randn(N, Fm, device=dev).bfloat16()
        add("gemm_tcgen05 dgrad (B n-major)", f"{N}x{D}x{Fm}", time_ms(lambda: ops.gemm_bf16(dy, b, None, 0, False, True)), 2.0 * N * Fm * D)
        add("cublas dgrad (twin)", f"{N}x{D}x{Fm}", time_ms(lambda: torch.matmul(dy, b)), 2.0 * N * Fm * D)
        add("gemm_tcgen05 wgrad (both mn-major)", f"{Fm}x{D}x{N}", time_ms(lambda: ops.gemm_bf16(dy, a, None, 0, True, True)), 2.0 * N * Fm * D)
        add("cublas wgrad (twin)", f"{Fm}x{D}x{N}", time_ms(lambda: torch.matmul(dy.T, a)), 2.0 * N * Fm * D)
        prev = ops.gemm_pair_mode(1 - ops.gemm_pair_mode(-1))
        tagp = "CTA pairs" if prev == 0 else "single-CTA tiles"
        add(f"gemm_tcgen05 nt +gelu(+pre), {tagp}", f"{N}x{Fm}x{D}", time_ms(lambda: ops.gemm_bf16_gelu_pre(a, b, None)), 2.0 * N * Fm * D)
        add(f"gemm_tcgen05 dgrad, {tagp}", f"{N}x{D}x{Fm}", time_ms(lambda: ops.gemm_bf16(dy, b, None, 0, False, True)), 2.0 * N * Fm * D)
        add(f"gemm_tcgen05 wgrad, {tagp}", f"{Fm}x{D}x{N}", time_ms(lambda: ops.gemm_bf16(dy, a, None, 0, True, True)), 2.0 * N * Fm * D)
        ops.gemm_pair_mode(prev)
        del a, b, dy
    if want("attention"):
        heads = args.heads or (2 if args.quick else H)
        q, k, v = (torch.randn(1, N, heads, HD, device=dev).bfloat16() for _ in range(3))
        fl = 4.0 * N * N * HD * heads
        scale = 1 / math.sqrt(HD)
        add("fa_fwd tcgen05", f"S={N} H={heads} hd=128", time_ms(lambda: ops.fa_fwd(q, k, v, scale), iters=3, warmup=1), fl)
        if not args.no_twin:
            add("cudnn sdpa fwd (twin)", f"S={N} H={heads}", time_ms(lambda: F_ops._sdpa(q, k, v, scale), iters=3, warmup=1), fl)
        if args.variants and hasattr(ops, "fa_fwd_variant"):
            for var in (1, 2, 3, 4, 5, 6, 9, 10, 11):
                add(f"fa_fwd tcgen05 variant {var}", f"S={N} H={heads}",
                    time_ms(lambda: ops.fa_fwd_variant(q, k, v, scale, var), iters=3, warmup=1), fl)
        if hasattr(ops, "fa_bwd"):
            o, lse = ops.fa_fwd(q, k, v, scale)
            do = torch.randn_like(o)
            add("fa_bwd tcgen05 two-kernel (7 GEMM)", f"S={N} H={heads}",
                time_ms(lambda: ops.fa_bwd_variant(do, q, k, v, o, lse, scale, 1), iters=3, warmup=1), 2.5 * fl)
            add("fa_bwd tcgen05 single-pass, 128x64 sub-tiles (5 GEMM)", f"S={N} H={heads}",
                time_ms(lambda: ops.fa_bwd_variant(do, q, k, v, o, lse, scale, 2), iters=3, warmup=1), 2.5 * fl)
            add("fa_bwd tcgen05 single-pass, 128x128 tiles (5 GEMM)", f"S={N} H={heads}",
                time_ms(lambda: ops.fa_bwd_variant(do, q, k, v, o, lse, scale, 3), iters=3, warmup=1), 2.5 * fl)
        if hasattr(ops, "fa_jvp"):
            tq, tk, tv = (torch.randn_like(t) for t in (q, k, v))
            # useful work: S, tS (2 GEMMs), P V (forward), A V, P tV = 6 GEMM units of 2 S^2 D H each
            add("fa_jvp tcgen05 (forward + tangent pass)", f"S={N} H={heads}",
                time_ms(lambda: ops.fa_jvp(q, k, v, tq, tk, tv, scale), iters=3, warmup=1), 3.0 * fl)
        if hasattr(ops, "fa_fwd_na") and N == 84480:
            # neighbourhood attention at the reference's tuned 720p configuration: grid 24 x 44 x 80 tokens, window (24, 12, 24),
            # stride (1, 4, 8); "useful" FLOPs count visible keys only (window volume per query)
            from ..modules import neighborhood_attn as na
            vs, win, st = (24, 44, 80), (24, 12, 24), (1, 4, 8)
            plan = na.tile_plan(vs, win, st, (False, False, False), q.device)
            qt, kt, vt = q, k, v                                        # natural token order: the kernel tiles by itself
            fl_na = 4.0 * N * (win[0] * win[1] * win[2]) * HD * heads
            add("fa_fwd_na tcgen05 (tile-sparse neighbourhood attention)", f"grid={vs} window={win} stride={st} H={heads}",
                time_ms(lambda: ops.fa_fwd_na(qt, kt, vt, scale, plan.kv_idx, plan.kv_cnt, plan.bt, plan.bh, plan.bw), iters=3, warmup=1),
                fl_na, note=f"visited key tiles: {plan.visited_fraction:.3f} of dense; dense fa_fwd above is the baseline")
        if not args.no_twin:
            qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
            og = F_ops._sdpa(qg, kg, vg, scale)
            dog = torch.randn_like(og)
            add("cudnn sdpa bwd (twin)", f"S={N} H={heads}",
                time_ms(lambda: torch.autograd.grad(og, (qg, kg, vg), dog, retain_graph=True), iters=3, warmup=1), 2.5 * fl)
        kc, vc = (torch.randn(1, 512, heads, HD, device=dev).bfloat16() for _ in range(2))
        add("fa_fwd tcgen05 cross (Skv=512)", f"Sq={N} H={heads}", time_ms(lambda: ops.fa_fwd(q, kc, vc, scale)), 4.0 * N * 512 * HD * heads)
        if not args.no_twin:
            add("cudnn sdpa cross (twin)", f"Sq={N} H={heads}", time_ms(lambda: F_ops._sdpa(q, kc, vc, scale)), 4.0 * N * 512 * HD * heads)
        if args.variants:
            for var in (7, 8, 4, 1):
                add(f"fa_fwd tcgen05 cross variant {var}", f"Sq={N} H={heads}",
                    time_ms(lambda: ops.fa_fwd_variant(q, kc, vc, scale, var)), 4.0 * N * 512 * HD * heads)
        if args.reference:
            ref_attn = _load_reference_module("cosmos_predict2/_src/predict2/networks/attention.py", "reference_attention")
            if ref_attn is None:
                print(json.dumps({"reference": "baseline/_ref is absent"}), flush=True)
            else:
                add("reference attention() dispatcher fwd", f"S={N} H={heads}",
                    time_ms(lambda: ref_attn.attention(q, k, v, softmax_scale=scale), iters=3, warmup=1), fl)
                add("reference attention() dispatcher cross (Skv=512)", f"Sq={N} H={heads}",
                    time_ms(lambda: ref_attn.attention(q, kc, vc, softmax_scale=scale)), 4.0 * N * 512 * HD * heads)
            try:
                ref_jvp = _load_reference_module("cosmos_predict2/_src/predict2/utils/flash_attention_jvp_triton.py", "reference_jvp")
            except Exception as e:   # the file imports triton and flash_attn
                ref_jvp = None
                print(json.dumps({"reference_jvp": f"import failed: {type(e).__name__}: {e}"}), flush=True)
            if ref_jvp is not None:
                # the Triton kernel wants [B, H, S, D]; same tensors, transposed views made contiguous once outside the timing
                qh, kh, vh = (t.transpose(1, 2).contiguous() for t in (q, k, v))
                tqh, tkh, tvh = (torch.randn_like(t) for t in (qh, kh, vh))
                add("reference Triton JVP attention (forward + tangent)", f"S={N} H={heads}",
                    time_ms(lambda: ref_jvp.attention(qh, kh, vh, tqh, tkh, tvh, False, scale), iters=3, warmup=2), 3.0 * fl)
                del qh, kh, vh, tqh, tkh, tvh
        del q, k, v
    if want("elementwise"):
        x = torch.randn(1, T, L, D, device=dev).bfloat16()
        y = torch.randn_like(x)
        sh, sc, g = (torch.randn(1, T, D, device=dev) for _ in range(3))
        nb = x.numel() * 2
        xf = x.view(-1, D)
        add("ln_modulate_fwd", f"{T * L}x{D}", time_ms(lambda: ops.ln_modulate_fwd(xf, sh.view(-1, D), sc.view(-1, D), L, 1e-6)), bytes_=2 * nb)
        yy, mean, rstd = ops.ln_modulate_fwd(xf, sh.view(-1, D), sc.view(-1, D), L, 1e-6)
        add("ln_modulate_bwd", f"{T * L}x{D}", time_ms(lambda: ops.ln_modulate_bwd(y.view(-1, D), xf, mean, rstd, sc.view(-1, D), L)), bytes_=3 * nb)
        add("torch LN+mod fwd (twin)", f"{T * L}x{D}",
            time_ms(lambda: torch.nn.functional.layer_norm(x, (D,), eps=1e-6) * (1 + sc.bfloat16().unsqueeze(2)) + sh.bfloat16().unsqueeze(2)), bytes_=2 * nb)
        add("gate_residual_fwd", f"{T * L}x{D}", time_ms(lambda: ops.gate_residual_fwd(xf, g.view(-1, D), y.view(-1, D), L)), bytes_=3 * nb)
        add("gate_residual_bwd", f"{T * L}x{D}", time_ms(lambda: ops.gate_residual_bwd(xf, g.view(-1, D), y.view(-1, D), L)), bytes_=3 * nb)
        add("torch x+g*y (twin)", f"{T * L}x{D}", time_ms(lambda: x + g.bfloat16().unsqueeze(2) * y), bytes_=3 * nb)
        q = torch.randn(1, T * L, H, HD, device=dev).bfloat16()
        w = torch.ones(HD, device=dev)
        ang = torch.rand(T * L, HD, device=dev)
        rope = F_ops.RopeTable(ang)
        cos, sin = rope.cos_sin()
        add("rmsnorm_rope_fwd", f"{T * L}x{H}x{HD}", time_ms(lambda: ops.rmsnorm_rope_fwd(q, w, cos, sin, 1e-6)), bytes_=2 * q.numel() * 2 + 2 * cos.numel() * 4)
        yq, rs = ops.rmsnorm_rope_fwd(q, w, cos, sin, 1e-6)
        add("rmsnorm_rope_bwd", f"{T * L}x{H}x{HD}", time_ms(lambda: ops.rmsnorm_rope_bwd(q, q, w, rs, cos, sin)), bytes_=3 * q.numel() * 2)
        h = torch.randn(T * L, Fm, device=dev).bfloat16()
        add("gelu_bwd", f"{T * L}x{Fm}", time_ms(lambda: ops.gelu_bwd(h, h)), bytes_=3 * h.numel() * 2)
        # forward-mode (value + tangent) variants: two tensors in, two out
        add("ln_modulate_jvp", f"{T * L}x{D}", time_ms(lambda: ops.ln_modulate_jvp(xf, y.view(-1, D), sh.view(-1, D), sc.view(-1, D),
                                                                                  sh.view(-1, D), sc.view(-1, D), L, 1e-6)), bytes_=4 * nb)
        add("rmsnorm_rope_jvp", f"{T * L}x{H}x{HD}", time_ms(lambda: ops.rmsnorm_rope_jvp(q, q, w, cos, sin, 1e-6)), bytes_=4 * q.numel() * 2)
        del x, y, q, h
    if want("skinny"):
        # AdaLN-LoRA modulation MLPs of the 2B network: rows = batch x latent frames, D -> 256 -> 3D, bf16 weights, fp32 math
        R, r = 2 * T, 256
        emb = torch.randn(R, D, device=dev)
        lora = torch.randn(R, 3 * D, device=dev)
        for Z, tag in ((3, "one block"), (84, "all 28 blocks in one launch")):
            w1 = [(torch.randn(r, D, device=dev) * 0.02).bfloat16() for _ in range(Z)]
            w2 = [(torch.randn(3 * D, r, device=dev) * 0.02).bfloat16() for _ in range(Z)]
            wb = Z * (r * D + 3 * D * r) * 2.0

            def two_stage():
                return F_ops.skinny_linears(F_ops.skinny_linears(emb, w1, silu=True), w2, add=lora)

            def torch_twin():
                a = torch.nn.functional.silu(emb)
                return [torch.nn.functional.linear(torch.nn.functional.linear(a, w1[z].float()), w2[z].float()) + lora for z in range(Z)]

            add(f"skinny_bgemm x2 (AdaLN-LoRA, {tag})", f"Z={Z} rows={R} {D}->{r}->{3 * D}", time_ms(two_stage), bytes_=wb)
            add(f"torch fp32 linears (twin, {tag})", f"Z={Z} rows={R}", time_ms(torch_twin), bytes_=wb)
            del w1, w2
    if want("sampler"):
        # state updates of the sampling loop on the batched cond / uncond latent [2, 16, 24, 88, 160] fp32 (21.6 MB per tensor,
        # smaller than L2: the flush between iterations makes every operand come from HBM)
        from . import ref as ref_ops
        shape = (2, 16, 24, 88, 160)
        xs = [torch.randn(shape, device=dev) for _ in range(4)]
        cs = [0.9, -0.3, 0.2, 0.05]
        nbt = xs[0].numel() * 4.0
        add("lincomb (4 operands: corrector update)", "2x16x24x88x160 fp32", time_ms(lambda: F_ops.lincomb(xs, cs)), bytes_=5 * nbt)
        add("torch term by term (twin)", "4 operands", time_ms(lambda: ref_ops.lincomb(xs, cs)), bytes_=5 * nbt)
        mask = torch.zeros(2, 1, 24, 88, 160, device=dev)
        mask[:, :, :2] = 1
        flag = torch.ones(2, 1, 1, 1, 1, device=dev)
        add("frame_blend -> bf16 (conditioning frames in)", "2x16x24x88x160", time_ms(
            lambda: F_ops.frame_blend(xs[0], xs[1], None, mask, flag, out_dtype=torch.bfloat16)), bytes_=2.5 * nbt + mask.numel() * 4.0)
        add("torch blend + cast (twin)", "", time_ms(
            lambda: ref_ops.frame_blend(xs[0], xs[1], None, mask, flag, out_dtype=torch.bfloat16)), bytes_=2.5 * nbt + mask.numel() * 4.0)
        add("frame_blend (velocity of conditioning frames)", "2x16x24x88x160", time_ms(
            lambda: F_ops.frame_blend(xs[0], xs[1], xs[2], mask)), bytes_=4 * nbt + mask.numel() * 4.0)
        add("torch blend (twin)", "", time_ms(lambda: ref_ops.frame_blend(xs[0], xs[1], xs[2], mask)), bytes_=4 * nbt + mask.numel() * 4.0)
        del xs
    if want("conv"):
        # causal 3 x 3 x 3 convolutions of the Wan2.1 VAE decoder at 720p (channels-last activations, 2 cached + 4 new frames in,
        # 4 frames out), next to the cuDNN convolution of the same layer on NCTHW tensors
        from ..models.vae_wan_cl import ConvCL, _causal3_taps
        div = 2 if (args.quick or args.seq) else 1
        for C, Hh, Ww, tag in ((384, 176 // div, 320 // div, "stage 1"), (192, 352 // div, 640 // div, "stage 2"), (96, 704 // div, 1280 // div, "stage 3")):
            wt = torch.randn(C, 27, C, device=dev) * (27 * C) ** -0.5
            conv = ConvCL(wt, torch.zeros(C, device=dev), _causal3_taps(3, 3, 3), dev)
            xin = torch.randn(6, Hh, Ww, C, device=dev).bfloat16()
            fl = 2.0 * 27 * C * C * 4 * Hh * Ww
            add(f"conv_cl 3x3x3 causal ({tag})", f"C={C} {4}x{Hh}x{Ww}", time_ms(lambda: conv(xin, 4)), fl)
            if not args.no_twin:
                w5 = wt.view(C, 3, 3, 3, C).permute(0, 4, 1, 2, 3).contiguous().bfloat16()
                x5 = xin.permute(3, 0, 1, 2).unsqueeze(0).contiguous()
                add(f"cudnn conv3d (twin, {tag})", f"C={C}", time_ms(lambda: torch.nn.functional.conv3d(x5, w5, padding=(0, 1, 1))), fl)
            del wt, conv, xin
    if want("optimizer"):
        n = 69_000_000 if not args.quick else 8_000_000
        g16 = torch.randn(n, device=dev).bfloat16()
        g32 = torch.empty(n, device=dev)
        ss = torch.zeros(1, device=dev)
        add("grad_cast_norm", f"{n}", time_ms(lambda: ops.grad_cast_norm(g16, g32, ss, 1.0)), bytes_=6 * n)
        ms_, m_, v_, e_ = (torch.zeros(n, device=dev) for _ in range(4))
        o16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
        clip = torch.ones(1, device=dev)
        add("adamw_ema_shard", f"{n}", time_ms(lambda: ops.adamw_ema_shard(ms_, g32, m_, v_, e_, o16, clip, 1e-4, 0.9, 0.999, 1e-8, 1e-3, 1, 0.99)),
            bytes_=(4 * 5 + 4 * 4 + 2) * n)
    err = ops.kernel_error(torch.cuda.current_device(), True)
    print(json.dumps({"kernel_error": int(err), "peaks": pk}))
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"rows": rows, "peaks": pk, "kernel_error": int(err)}, f, indent=1)


if __name__ == "__main__":
    main()
