"""Single-kernel runs for timing and profiling.

    python -m torchless_rs_b200.measure gemm M N K MODE [--iters I]
    python -m torchless_rs_b200.measure attn-decode BATCH CONTEXT [--iters I]
    python -m torchless_rs_b200.measure attn-prefill TOKENS [--iters I]
    python -m torchless_rs_b200.measure elementwise TOKENS [--iters I]
    python -m torchless_rs_b200.measure step BATCH CONTEXT PREFILL_TOKENS [--layers L] [--iters I]
    python -m torchless_rs_b200.measure timeline BATCH CONTEXT [--layers L]

Each prints the mean device time per launch (CUDA events, after warm-up; the weights
or the cache are larger than the L2 cache or rotated so that they come from HBM) and
the bandwidth or arithmetic rate that this time means.  Sizes other than the ones
given default to those of Mistral 7B (32 heads, 8 key/value heads, head size 128).

`step` runs whole steps of the engine, kernel by kernel (no CUDA graph), on a model with
the layer sizes of Mistral 7B, random weights and L layers: I prefill steps of
PREFILL_TOKENS tokens, then I decode steps of BATCH sequences that hold CONTEXT tokens of
random cache content.  It is the small case for a profiler's list of launches: which kernels
a step consists of and how its time divides among them.
"""
from __future__ import annotations

import argparse
import math

import torch


def _time(fn, iters: int) -> float:
    """Mean microseconds per call.  The calls are recorded into one CUDA graph and the graph
    is replayed, so the host's launch cost (some ten microseconds per call from Python) does
    not bound what is measured."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (3 * iters)   # microseconds


def gemm(M: int, N: int, K: int, mode: int, iters: int) -> None:
    from .csrc.gemm_bf16 import GemmBf16
    g = GemmBf16.get()
    rows = 2 * N if mode == 2 else N
    copies = max(2, int(400e6 // (rows * K * 2)) + 1)     # rotate weights: more than the L2 holds
    ws = [torch.randn((rows, K), device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn((M, K), device="cuda", dtype=torch.bfloat16)
    out = torch.zeros((M, N), device="cuda", dtype=torch.float32 if mode in (0, 1) else torch.bfloat16)
    state = {"i": 0}

    def run():
        assert g.run(x, ws[state["i"] % copies], out, mode), "shape not taken by the tensor-core kernel"
        state["i"] += 1
    us = _time(run, iters)
    print(f"gemm M={M} N={N} K={K} mode={mode}: {us:.2f} us, "
          f"{rows * K * 2 / us / 1e3:.0f} GB/s of weights, {2.0 * M * rows * K / us / 1e6:.1f} TFLOP/s, "
          f"error word {g.take_error()}")


def _paged(B: int, ctx: int, nkv: int, hd: int):
    pages = (ctx + 63) // 64
    kp = torch.randn((B * pages, nkv, 64, hd), device="cuda", dtype=torch.bfloat16)
    vp = torch.randn((B * pages, nkv, hd, 64), device="cuda", dtype=torch.bfloat16)
    table = torch.arange(B * pages, dtype=torch.int32, device="cuda").view(B, pages)
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    return kp, vp, table, slot


def attn_decode(B: int, ctx: int, iters: int, nh=32, nkv=8, hd=128) -> None:
    from .csrc import attention_bf16
    from .csrc.attention_bf16 import AttentionBf16
    from .parts.runtime import Workspace
    decode_splits = attention_bf16.decode_splits
    att, ws = AttentionBf16.get(hd), Workspace(torch.device("cuda"))
    kp, vp, table, slot = _paged(B, ctx, nkv, hd)
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn((B, nh * hd), device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    n = decode_splits(B, nkv, ctx, None)
    us = _time(lambda: att.decode(q, kp, vp, out, lens, slot, table, nh, nkv, None,
                                  1 / math.sqrt(hd), n, ws), iters)
    byts = 2.0 * B * ctx * nkv * hd * 2
    print(f"attn-decode B={B} context={ctx} splits={n}: {us:.2f} us (both kernels), {byts / us / 1e3:.0f} GB/s of cache")


def attn_prefill(T: int, iters: int, nh=32, nkv=8, hd=128) -> None:
    from .csrc.attention_bf16 import AttentionBf16
    att = AttentionBf16.get(hd)
    kp, vp, table, slot = _paged(1, T, nkv, hd)
    start = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    lens = torch.tensor([T], dtype=torch.int32, device="cuda")
    q = torch.randn((T, nh * hd), device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    for variant in ("tc", "tma"):
        us = _time(lambda: att.prefill(q, kp, vp, out, start, lens, slot, table, 1, T, nh, nkv, None,
                                       1 / math.sqrt(hd), variant=variant), iters)
        print(f"attn-prefill tokens={T} kernel={variant}: {us:.2f} us, "
              f"{2.0 * nh * hd * T * T / us / 1e6:.1f} TFLOP/s (causal half counted), error word {att.take_error()}")


def elementwise(T: int, iters: int, H=4096, nh=32, nkv=8, hd=128) -> None:
    """The norm kernel and the rotation + cache write kernel of a prefill step of T tokens, each with inputs
    rotated through more than the L2 cache holds and with one input over and over (as in a step, where the
    kernel before has just written it)."""
    from .csrc import ops
    o = ops.core_ops(torch.bfloat16)
    copies = max(2, int(400e6 // (T * H * 4)) + 1)
    xs = [torch.randn((T, H), device="cuda") for _ in range(copies)]
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y = torch.empty((T, H), device="cuda", dtype=torch.bfloat16)
    st = {"i": 0}

    def norm(rotate):
        o.rmsnorm(xs[st["i"] % copies if rotate else 0], w, 1e-5, y)
        st["i"] += 1
    byts = T * H * 6.0
    for rotate in (True, False):
        us = _time(lambda: norm(rotate), iters)
        print(f"rmsnorm {T} x {H}, {'inputs from HBM' if rotate else 'input in L2'}: {us:.2f} us, {byts / us / 1e3:.0f} GB/s")
    cols = (nh + 2 * nkv) * hd
    copies = max(2, int(400e6 // (T * cols * 4)) + 1)
    qkvs = [torch.randn((T, cols), device="cuda") for _ in range(copies)]
    q = torch.empty((T, nh * hd), device="cuda", dtype=torch.bfloat16)
    pages = (T + 63) // 64
    kp = torch.zeros((pages, nkv, 64, hd), device="cuda", dtype=torch.bfloat16)
    vp = torch.zeros((pages, nkv, hd, 64), device="cuda", dtype=torch.bfloat16)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    half = hd // 2
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(half, dtype=torch.float64) / half)).float().cuda()

    def rope(rotate):
        o.rope_cache_write(qkvs[st["i"] % copies if rotate else 0], q, kp, vp, pos, seq, slot, table, inv, 0, nh, nkv, hd)
        st["i"] += 1
    byts = T * cols * 6.0
    for rotate in (True, False):
        us = _time(lambda: rope(rotate), iters)
        print(f"rotation + cache write, {T} tokens, {'inputs from HBM' if rotate else 'input in L2'}: {us:.2f} us, "
              f"{byts / us / 1e3:.0f} GB/s")


MISTRAL_7B_SIZES = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_size": 4096,
    "intermediate_size": 14336, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 32000, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "sliding_window": 4096,
    "max_position_embeddings": 32768, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
}
# the layer sizes of the two larger workloads that bench.py names (Mistral NeMo 12B, Mistral Small 22B)
MODEL_SIZES = {
    "mistral7b": MISTRAL_7B_SIZES,
    "nemo12b": dict(MISTRAL_7B_SIZES, hidden_size=5120, vocab_size=131072, rope_theta=1e6, sliding_window=None,
                    max_position_embeddings=131072),
    "small22b": dict(MISTRAL_7B_SIZES, hidden_size=6144, num_attention_heads=48, intermediate_size=16384,
                     vocab_size=32768, rope_theta=1e6, sliding_window=None),
}
SIZES = MISTRAL_7B_SIZES   # what `step` and `timeline` build; --model chooses


# Layer sizes at which the Kikopel kernels are measured: the width, heads and feed-forward of a 1B- and a
# 7B-class decoder, latent ranks and head sizes as published latent-attention models have them, a recurrent
# state of 128 x 128 per head.
KIKOPEL_SIZES = {
    "1b": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, q_rank=768, kv_rank=512, window=4096, ff=5632,
               r_heads=16, r_dim=128, r_vdim=128, vocab=32000),
    "7b": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, q_rank=1536, kv_rank=512, window=4096, ff=14336,
               r_heads=32, r_dim=128, r_vdim=128, vocab=32000),
}


def kikopel_config(size: str, layers: int) -> dict:
    """config.json of a Kikopel model of `layers` layers at these sizes: attention, recurrence, attention,
    attention, and so on."""
    z = KIKOPEL_SIZES[size]
    att = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": z["ff"]},
           "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"],
                     "q_rank": z["q_rank"], "kv_rank": z["kv_rank"], "mask": {"size": z["window"]},
                     "rot": {"base": 500000.0, "dims": z["rot"]}, "scale": 1.0 / math.sqrt(z["dim"] + z["rot"])}}
    rec = {"type": "hgrn2", "mlp": {"kind": "dense", "ff": z["ff"]},
           "mixer": {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"]}}
    return {"architecture": "Kikopel", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-5},
            "residual_mult": 0.6, "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 8191, "mul_cur": 131}},
            "layers": [rec if i % 4 == 1 else att for i in range(layers)], "max_position_embeddings": 32768}


def mistral_like(size: str, layers: int) -> dict:
    """The closest existing model at equal size: Mistral with the same width, heads, feed-forward and window."""
    z = KIKOPEL_SIZES[size]
    return dict(MISTRAL_7B_SIZES, num_hidden_layers=layers, hidden_size=z["width"], num_attention_heads=z["heads"],
                num_key_value_heads=max(1, z["heads"] // 4), head_dim=128, intermediate_size=z["ff"],
                vocab_size=z["vocab"], sliding_window=z["window"], max_position_embeddings=32768)


def kikopel_kernels(size: str, T: int, B: int, ctx: int, iters: int, file=None) -> list:
    """Every kernel of the Kikopel design alone at the sizes `size`, for a prompt of T tokens and for a decode
    step of B sequences at a context of `ctx`, beside the like kernel of the Mistral path at equal sizes.
    Returns rows (name, case, microseconds, fraction of the roofline, what bounds it) and prints them.  The
    roofline of a kernel is the larger of its algorithmic bytes over the measured copy bandwidth and its
    FLOPs over the measured bf16 tensor rate (also for kernels that run on CUDA cores: the like kernels of
    the Mistral path are on tensor cores, and the comparison is against what the hardware could do)."""
    import json
    import os
    from .csrc import ops
    from .csrc.attention_bf16 import AttentionBf16
    z = KIKOPEL_SIZES[size]
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.isfile(pk):
        peaks.update(json.load(open(pk)))
    o = ops.core_ops(torch.bfloat16)
    dev, bf = "cuda", torch.bfloat16
    H, rank, rot, vdim, W = z["heads"], z["kv_rank"], z["rot"], z["vdim"], z["width"]
    width = rank + rot
    rows = []

    def report(name, case, us, byts, flops):
        t_mem, t_fl = byts / (peaks["hbm_gbs"] * 1e3), flops / (peaks["bf16_tflops"] * 1e6)     # microseconds
        frac = max(t_mem, t_fl) / us
        rows.append({"kernel": name, "case": case, "us": round(us, 2), "roofline_frac": round(frac, 4),
                     "bound": "memory" if t_mem >= t_fl else "tensor"})
        print(f"{name:28s} {case:22s} {us:10.2f} us   {frac:7.4f} of the roofline ({rows[-1]['bound']})", file=file)

    inv = torch.tensor([500000.0 ** (-2.0 * i / rot) for i in range(rot // 2)], device=dev)
    for case, n_tok, seqs, past in ((f"prompt {T}", T, 1, 0), (f"decode {B} x {ctx}", B, B, ctx - 1)):
        per = n_tok // seqs
        pages_per = (past + per + 63) // 64
        pos = torch.cat([torch.arange(past, past + per, dtype=torch.int32) for _ in range(seqs)]).to(dev)
        seq = torch.arange(seqs, dtype=torch.int32).repeat_interleave(per).to(dev)
        slot = torch.arange(seqs, dtype=torch.int32, device=dev)
        start = (torch.arange(seqs + 1, dtype=torch.int32) * per).to(dev)
        table = torch.arange(seqs * pages_per, dtype=torch.int32, device=dev).view(seqs, pages_per)
        seen = sum(min(p + 1, z["window"]) for p in range(past, past + per)) * seqs      # (query, key) pairs
        # --- the attention through latents, and Mistral's attention at equal heads
        pages = torch.randn((seqs * pages_per, 64, width), device=dev, dtype=bf)
        q = torch.randn((n_tok, H * width), device=dev) * 0.1
        mix = torch.empty((n_tok, H, rank), device=dev)
        us = _time(lambda: o.latent_attn(q, width, q, width, rank, pages, mix, pos, seq, slot, table, inv, H, rank,
                                         rot, rot, z["window"], 0.04), max(2, iters // 8) if n_tok > 64 else iters)
        cache_b = 2.0 * seqs * min(past + per, z["window"]) * width
        report("latent_attn", case, us, cache_b + n_tok * H * (width + rank) * 4.0, 2.0 * H * seen * (width + rank))
        nkv = max(1, H // 4)
        att = AttentionBf16.get(128)
        kp, vp, tab2, slot2 = _paged(seqs, past + per, nkv, 128)
        qm = torch.randn((n_tok, H * 128), device=dev, dtype=bf)
        om = torch.empty_like(qm)
        lens = torch.full((seqs,), past + per, dtype=torch.int32, device=dev)
        if seqs == 1:
            us = _time(lambda: att.prefill(qm, kp, vp, om, start, lens, slot2, tab2, 1, n_tok, H, nkv, z["window"],
                                           0.088, variant="tc"), iters)
        else:
            from .csrc import attention_bf16
            from .parts.runtime import Workspace
            ws = Workspace(torch.device("cuda"))
            n = attention_bf16.decode_splits(seqs, nkv, past + per, z["window"])
            us = _time(lambda: att.decode(qm, kp, vp, om, lens, slot2, tab2, H, nkv, z["window"], 0.088, n, ws), iters)
        report("  like: attention (Mistral)", case, us,
               2.0 * seqs * min(past + per, z["window"]) * nkv * 128 * 2 + n_tok * H * 128 * 4.0, 4.0 * H * 128 * seen)
        # --- per-head value up-projection with the gate, beside a tensor-core product of the same FLOPs
        wuv = torch.randn((H, vdim, rank), device=dev, dtype=bf) * 0.02
        gate = torch.randn((n_tok, H * vdim), device=dev)
        og = torch.empty((n_tok, H * vdim), device=dev, dtype=bf)
        us = _time(lambda: o.headwise_gemm(mix.view(n_tok, H * rank), rank, wuv, og, vdim, gate=gate), iters)
        report("headwise_gemm (values, gate)", case, us,
               H * vdim * rank * 2.0 + n_tok * H * (rank * 4.0 + vdim * 6.0), 2.0 * n_tok * H * vdim * rank)
        # --- what is written per token, beside Mistral's rotation + cache write
        dq = torch.randn((n_tok, z["q_rank"] + width), device=dev)
        cq = torch.empty((n_tok, z["q_rank"]), device=dev, dtype=bf)
        wq, wc = torch.ones(z["q_rank"], device=dev), torch.ones(rank, device=dev)
        us = _time(lambda: o.latent_prep(dq[:, :z["q_rank"]], dq[:, z["q_rank"]:], wq, wc, 1e-5, cq, pages, pos, seq,
                                         slot, table, inv, rank, rot, rot), iters)
        report("latent_prep", case, us, n_tok * ((z["q_rank"] + width) * 4.0 + (z["q_rank"] + width) * 2.0), 0.0)
        qkv = torch.randn((n_tok, (H + 2 * nkv) * 128), device=dev)
        inv128 = torch.tensor([1e6 ** (-i / 64.0) for i in range(64)], device=dev)
        us = _time(lambda: o.rope_cache_write(qkv, qm, kp, vp, pos, seq, slot2, tab2, inv128, 0, H, nkv, 128), iters)
        report("  like: rope_cache_write", case, us, n_tok * (H + 2 * nkv) * 128 * 6.0, 0.0)
        # --- the recurrence (no like kernel: the nearest is decode attention, which also streams per-sequence
        # memory; its algorithmic bytes are the projections and, once per sequence, the state in and out)
        rh, rd, rv = z["r_heads"], z["r_dim"], z["r_vdim"]
        zz = torch.randn((n_tok, 2 * rh * rd + rh * rv), device=dev)
        state = torch.zeros((seqs, rh, rd, rv), device=dev)
        so = torch.empty((n_tok, rh * rv), device=dev)
        from .parts.runtime import Workspace as _Ws
        scan_ws = _Ws(torch.device("cuda"))
        bias, low = torch.zeros(rh * rd, device=dev), torch.full((rh * rd,), 0.5, device=dev)
        us = _time(lambda: o.gated_scan(zz, bias, low, state, so, start, slot, rh, rd, rv, workspace=scan_ws),
                   max(2, iters // 8) if n_tok > 64 else iters)
        report("gated_scan", case, us, n_tok * (2 * rh * rd + 2 * rh * rv) * 4.0 + seqs * rh * rd * rv * 8.0,
               4.0 * n_tok * rh * rd * rv)
        # --- the branch's norm + residual sum and the activation, beside Mistral's norm kernel
        y, x = torch.randn((n_tok, W), device=dev), torch.randn((n_tok, W), device=dev)
        xb = torch.empty((n_tok, W), device=dev, dtype=bf)
        g1 = torch.ones(1, device=dev)
        us = _time(lambda: o.branch_norm_add(y, g1, 0.6, 1e-5, x, xb), iters)
        report("branch_norm_add", case, us, n_tok * W * 14.0, 0.0)
        zf = torch.randn((n_tok, z["ff"]), device=dev)
        af = torch.empty((n_tok, z["ff"]), device=dev, dtype=bf)
        co = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev)
        us = _time(lambda: o.poly_norm(zf, co, 1e-5, af), iters)
        report("poly_norm", case, us, n_tok * z["ff"] * 6.0, 0.0)
        wn = torch.ones(W, device=dev, dtype=bf)
        us = _time(lambda: o.rmsnorm(x, wn, 1e-5, xb), iters)
        report("  like: rmsnorm", case, us, n_tok * W * 6.0, 0.0)
    return rows


# Layer sizes at which the Tovapel kernels are measured: the width, heads and feed-forward of a 1B- and a
# 7B-class decoder; four residual streams; attention with a quarter as many key/value heads, a window of 4096
# that keeps the first four keys; gated linear attention with keys of half and values of the full width;
# every other layer sixteen experts of a quarter of the dense inner size, four chosen, two pass-through outputs.
TOVAPEL_SIZES = {
    "1b": dict(width=2048, streams=4, heads=16, kv_heads=4, dim=128, vdim=128, window=4096, keep_first=4, ff=5632,
               r_heads=16, r_dim=64, r_vdim=128, rank=16, experts=16, identity=2, top=4, e_ff=1408, vocab=32000),
    "7b": dict(width=4096, streams=4, heads=32, kv_heads=8, dim=128, vdim=128, window=4096, keep_first=4, ff=14336,
               r_heads=32, r_dim=64, r_vdim=128, rank=16, experts=16, identity=2, top=4, e_ff=3584, vocab=32000),
}


def tovapel_config(size: str, layers: int) -> dict:
    """config.json of a Tovapel model of `layers` layers at these sizes: dense and expert feed-forwards in turn."""
    z = TOVAPEL_SIZES[size]
    mixer = {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                      "scale": 1.0 / math.sqrt(z["dim"]), "softcap": 50.0,
                      "mask": {"size": z["window"], "keep_first": z["keep_first"]}},
             "right": {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"], "tau": 16.0, "rank": z["rank"]}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["e_ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"]}}
    return {"architecture": "Tovapel", "width": z["width"], "vocab": z["vocab"], "streams": z["streams"],
            "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "max_position_embeddings": 32768,
            "layers": [{"type": "parallel", "mixer": mixer, "mlp": moe if i % 2 else dense} for i in range(layers)]}


def tovapel_like(size: str, layers: int) -> dict:
    """The closest existing model at equal size: Mistral with the same width, heads, key/value heads,
    feed-forward and window."""
    z = TOVAPEL_SIZES[size]
    return dict(MISTRAL_7B_SIZES, num_hidden_layers=layers, hidden_size=z["width"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv_heads"], head_dim=128, intermediate_size=z["ff"],
                vocab_size=z["vocab"], sliding_window=z["window"], max_position_embeddings=32768)


def tovapel_kernels(size: str, T: int, B: int, ctx: int, iters: int, file=None) -> list:
    """Every kernel of the Tovapel design alone at the sizes `size`, for a prompt of T tokens and for a decode
    step of B sequences at a context of `ctx`, beside the like kernel of an existing model at equal sizes.
    Rows and roofline as `kikopel_kernels` defines them."""
    import json
    import os
    from .csrc import ops
    from .csrc.attention_bf16 import AttentionBf16
    from .csrc.gemm_bf16 import GemmBf16
    from .parts.runtime import Workspace
    from .parts.sink_attention import run_attention
    z = TOVAPEL_SIZES[size]
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.isfile(pk):
        peaks.update(json.load(open(pk)))
    o = ops.core_ops(torch.bfloat16)
    dev, bf = "cuda", torch.bfloat16
    H, G, dim, vdim, W, S = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["width"], z["streams"]
    rows = []

    def report(name, case, us, byts, flops):
        t_mem, t_fl = byts / (peaks["hbm_gbs"] * 1e3), flops / (peaks["bf16_tflops"] * 1e6)     # microseconds
        frac = max(t_mem, t_fl) / us
        rows.append({"kernel": name, "case": case, "us": round(us, 2), "roofline_frac": round(frac, 4),
                     "bound": "memory" if t_mem >= t_fl else "tensor"})
        print(f"{name:30s} {case:22s} {us:10.2f} us   {frac:7.4f} of the roofline ({rows[-1]['bound']})", file=file)

    ws = Workspace(torch.device("cuda"))
    for case, n_tok, seqs, past in ((f"prompt {T}", T, 1, 0), (f"decode {B} x {ctx}", B, B, ctx - 1)):
        per = n_tok // seqs
        few = max(2, iters // 8) if n_tok > 64 else iters
        pos = torch.cat([torch.arange(past, past + per, dtype=torch.int32) for _ in range(seqs)]).to(dev)
        seq = torch.arange(seqs, dtype=torch.int32).repeat_interleave(per).to(dev)
        start = (torch.arange(seqs + 1, dtype=torch.int32) * per).to(dev)
        seen = sum(min(p + 1, z["window"] + z["keep_first"]) for p in range(past, past + per)) * seqs
        kp, vp, table, slot = _paged(seqs, past + per, G, dim)
        lens = torch.full((seqs,), past + per, dtype=torch.int32, device=dev)
        # --- attention with sink, cap and kept first keys, beside Mistral's attention at equal heads
        q = torch.randn((n_tok, H * dim), device=dev, dtype=bf)
        out = torch.empty((n_tok, H * vdim), device=dev, dtype=bf)
        gate, sink = torch.randn((n_tok, H), device=dev), torch.zeros(H, device=dev)

        class _B:      # what the kernel choice reads of a step
            n_tokens, n_seqs, is_decode, max_len, seq_start, seq_len, seq_slot = n_tok, seqs, per == 1, past + per, start, lens, slot
        us = _time(lambda: run_attention(o, q, kp, vp, gate, sink, out, pos, seq, slot, table, H, G, dim, vdim,
                                         z["window"], z["keep_first"], 0.088, 50.0, _B, ws), few)
        cache_b = 2.0 * seqs * min(past + per, z["window"]) * G * (dim + vdim)
        report("sink_attn", case, us, cache_b + n_tok * H * (dim + vdim) * 2.0, 2.0 * H * (dim + vdim) * seen)
        att = AttentionBf16.get(128)
        om = torch.empty_like(q)
        if seqs == 1:
            us = _time(lambda: att.prefill(q, kp, vp, om, start, lens, slot, table, 1, n_tok, H, G, z["window"],
                                           0.088, variant="tc"), iters)
        else:
            from .csrc import attention_bf16
            n = attention_bf16.decode_splits(seqs, G, past + per, z["window"])
            us = _time(lambda: att.decode(q, kp, vp, om, lens, slot, table, H, G, z["window"], 0.088, n, ws), iters)
        report("  like: attention (Mistral)", case, us, cache_b + n_tok * H * 128 * 4.0, 4.0 * H * 128 * seen)
        # --- bias, query/key norm and cache write, beside Mistral's rotation + cache write
        cols = (H + G) * dim + G * vdim
        zq = torch.randn((n_tok, cols + H), device=dev)
        bias, wn = torch.zeros(cols, device=dev), torch.ones(dim, device=dev)
        us = _time(lambda: o.qk_norm_cache_write(zq, bias, wn, wn, 1e-5, q, kp, vp, pos, seq, slot, table, H, G, dim,
                                                 vdim), iters)
        report("qk_norm_cache_write", case, us, n_tok * cols * 6.0, 0.0)
        qkv = torch.randn((n_tok, (H + 2 * G) * 128), device=dev)
        inv128 = torch.tensor([1e6 ** (-i / 64.0) for i in range(64)], device=dev)
        us = _time(lambda: o.rope_cache_write(qkv, q, kp, vp, pos, seq, slot, table, inv128, 0, H, G, 128), iters)
        report("  like: rope_cache_write", case, us, n_tok * (H + 2 * G) * 128 * 6.0, 0.0)
        # --- the two recurrences: this design's beside the gated scan of the Kikopel path at equal state
        rh, rd, rv = z["r_heads"], z["r_dim"], z["r_vdim"]
        zz = torch.randn((n_tok, 2 * rh * rd + 2 * rh * rv), device=dev)
        za = torch.randn((n_tok, rh * rd), device=dev) + 3.0
        state = torch.zeros((seqs, rh, rd, rv), device=dev)
        so = torch.empty((n_tok, rh * rv), device=dev)
        ab = torch.zeros(rh * rd, device=dev)
        hd, hv = rh * rd, rh * rv
        us = _time(lambda: o.gla_scan(zz[:, :hd], zz[:, hd:2 * hd], zz[:, 2 * hd:2 * hd + hv], za, ab, 16.0, 0.125,
                                      state, so, start, slot, rh, rd, rv, workspace=ws), few)
        scan_b = n_tok * (3 * hd + 2 * hv) * 4.0 + seqs * hd * rv * 8.0
        report("gla_scan", case, us, scan_b, 4.0 * n_tok * hd * rv)
        z2 = torch.randn((n_tok, 2 * hd + hv), device=dev)
        low = torch.full((hd,), 0.5, device=dev)
        state.zero_()
        us = _time(lambda: o.gated_scan(z2, ab, low, state, so, start, slot, rh, rd, rv, workspace=ws), few)
        report("  like: gated_scan (Kikopel)", case, us, n_tok * (2 * hd + 2 * hv) * 4.0 + seqs * hd * rv * 8.0,
               4.0 * n_tok * hd * rv)
        gated = torch.empty((n_tok, hv), device=dev, dtype=bf)
        nw = torch.ones(rv, device=dev)
        us = _time(lambda: o.headnorm_silu_gate(so, nw, 1e-5, zz[:, 2 * hd + hv:], gated, rh, rv), iters)
        report("headnorm_silu_gate", case, us, n_tok * hv * 10.0, 0.0)
        # --- the streams, the branch norms, beside Mistral's norm kernel
        xs = torch.randn((n_tok, S, W), device=dev)
        y = torch.randn((n_tok, W), device=dev)
        a, b, M = torch.ones(S, device=dev) / S, torch.ones(S, device=dev), torch.eye(S, device=dev)
        w32 = torch.ones(W, device=dev)
        xb = torch.empty((n_tok, W), device=dev, dtype=bf)
        us = _time(lambda: o.hc_read_norm(xs, a, w32, 1e-5, xb), iters)
        report("hc_read_norm", case, us, n_tok * W * (4.0 * S + 2.0), 0.0)
        us = _time(lambda: o.hc_write(xs, M, b, y, next_read=(a, w32, 1e-5, xb)), iters)
        report("hc_write (+ next read, norm)", case, us, n_tok * W * (8.0 * S + 6.0), 0.0)
        y2 = torch.randn((n_tok, W), device=dev)
        x = torch.randn((n_tok, W), device=dev)
        us = _time(lambda: o.branch_norm_mean([y, y2], [w32, w32], 1e-5, x, accumulate=False), iters)
        report("branch_norm_mean", case, us, n_tok * W * 12.0, 0.0)
        wb = torch.ones(W, device=dev, dtype=bf)
        us = _time(lambda: o.rmsnorm(x, wb, 1e-5, xb), iters)
        report("  like: rmsnorm", case, us, n_tok * W * 6.0, 0.0)
        # --- the experts: choice and grouping, the two grouped products, the weighted sum; beside the
        # tensor-core product of the same FLOPs (all pairs through one expert's matrices)
        E, I, top, f = z["experts"], z["identity"], z["top"], z["e_ff"]
        zr = torch.randn((n_tok, E + I), device=dev)
        idx = torch.empty((n_tok, top), dtype=torch.int32, device=dev)
        wt = torch.empty((n_tok, top), device=dev)
        corr = torch.zeros(E + I, device=dev)
        off = torch.empty(E + 1, dtype=torch.int32, device=dev)
        row_token = torch.empty(n_tok * top, dtype=torch.int32, device=dev)
        row_of = torch.empty((n_tok, top), dtype=torch.int32, device=dev)

        def choose():
            o.moe_route(zr, corr, top, idx, wt)
            o.moe_plan(idx, E, off, row_token, row_of)
        us = _time(choose, iters)
        report("moe_route + moe_plan", case, us, n_tok * ((E + I) * 4.0 + top * 20.0), 0.0)
        xn = torch.randn((n_tok, W), device=dev, dtype=bf)
        w_up = torch.randn((E, 2 * f, W), device=dev, dtype=bf) * 0.02
        w_dn = torch.randn((E, W, f), device=dev, dtype=bf) * 0.02
        act = torch.empty((n_tok * top, f), device=dev, dtype=bf)
        yk = torch.empty((n_tok * top, W), device=dev)
        pairs = n_tok * top * E / (E + I)              # expected rows of real experts
        used = min(E, n_tok * top)                     # experts whose matrices a step must read
        us = _time(lambda: o.moe_gemm(xn, row_token, w_up, act, off, up=True, limit=7.0, alpha=1.702), few)
        report("moe_gemm (gate, up, act)", case, us, used * 2 * f * W * 2.0 + pairs * (W + f) * 2.0, 4.0 * pairs * f * W)
        us = _time(lambda: o.moe_gemm(act, None, w_dn, yk, off, up=False), few)
        report("moe_gemm (down)", case, us, used * f * W * 2.0 + pairs * (f * 2.0 + W * 4.0), 2.0 * pairs * f * W)
        gm = GemmBf16.get()
        rows_all = n_tok * top
        a_all = torch.randn((rows_all, W), device=dev, dtype=bf)
        c_all = torch.empty((rows_all, f), device=dev, dtype=bf)
        if gm.run(a_all, w_up[0], c_all, ops.MODE_SWIGLU):
            us = _time(lambda: gm.run(a_all, w_up[0], c_all, ops.MODE_SWIGLU), iters)
            report("  like: gemm_tc (gate, up, act)", case, us, 2 * f * W * 2.0 + rows_all * (W + f) * 2.0,
                   4.0 * rows_all * f * W)
        us = _time(lambda: o.moe_combine(yk, row_of, wt, xn, x, accumulate=False), iters)
        report("moe_combine", case, us, n_tok * W * (4.0 * top + 6.0), 0.0)
    return rows


# A decoder whose sublayers stand between two norms; differential attention (two maps of 64 per head over
# values of 128) and gated window attention (heads of 128, half of them rotated, unit-normed, capped) in
# turn; a squared-relu feed-forward of one and a half times the SwiGLU inner size (equal weights) and, every
# other layer, sixteen clamped experts in four groups of which two are kept, four chosen, plus a shared expert.
RUPASUN_SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, d_dim=64, dim=128, vdim=128, window=4096, like_ff=5632, ff=8448,
               experts=16, groups=4, keep=2, top=4, e_ff=1408, vocab=32000),
    "7b": dict(width=4096, heads=32, kv_heads=8, d_dim=64, dim=128, vdim=128, window=4096, like_ff=14336, ff=21504,
               experts=16, groups=4, keep=2, top=4, e_ff=3584, vocab=32000),
}


def rupasun_config(size: str, layers: int) -> dict:
    """config.json of a Rupasun model of `layers` layers at these sizes: the two mixers in turn, dense and
    expert feed-forwards in turn at half that pace (so every pairing occurs)."""
    z = RUPASUN_SIZES[size]
    diff = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["d_dim"], "vdim": z["vdim"],
            "scale": 1.0 / math.sqrt(z["d_dim"]), "diff": 0.2, "rot": {"dims": z["d_dim"], "base": 10000.0}}
    win = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": 1.0,
           "softcap": 50.0, "mask": {"size": z["window"]}, "rot": {"dims": z["dim"] // 2, "base": 10000.0}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["e_ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5,
                      "groups": {"count": z["groups"], "keep": z["keep"]}},
           "shared": {"ff": z["e_ff"], "limit": 7.0}}
    return {"architecture": "Rupasun", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-5},
            "max_position_embeddings": 32768,
            "layers": [{"type": "attention_2" if i % 2 else "attention", "mixer": win if i % 2 else diff,
                        "mlp": moe if (i // 2) % 2 else dense} for i in range(layers)]}


def rupasun_like(size: str, layers: int) -> dict:
    """The closest existing model at equal size: Mistral with the same width, heads, key/value heads and
    window, and a SwiGLU feed-forward of the dense layers' weight."""
    z = RUPASUN_SIZES[size]
    return dict(MISTRAL_7B_SIZES, num_hidden_layers=layers, hidden_size=z["width"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv_heads"], head_dim=128, intermediate_size=z["like_ff"],
                vocab_size=z["vocab"], sliding_window=z["window"], max_position_embeddings=32768)


def rupasun_kernels(size: str, T: int, B: int, ctx: int, iters: int, file=None) -> list:
    """Every kernel of the Rupasun design alone at the sizes `size`, for a prompt of T tokens and for a decode
    step of B sequences at a context of `ctx`, beside the like kernel of an existing model at equal sizes.
    Rows and roofline as `kikopel_kernels` defines them.  (The experts' grouped products, their plan and their
    weighted sum are the kernels that `tovapel_kernels` measures, at the same sizes.)"""
    import json
    import os
    from .csrc import ops
    from .csrc.attention_bf16 import AttentionBf16
    from .csrc.gemm_bf16 import GemmBf16
    from .parts.runtime import Workspace
    from .parts.sink_attention import run_attention
    z = RUPASUN_SIZES[size]
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.isfile(pk):
        peaks.update(json.load(open(pk)))
    o = ops.core_ops(torch.bfloat16)
    dev, bf = "cuda", torch.bfloat16
    H, G, dd, dim, vdim, W = z["heads"], z["kv_heads"], z["d_dim"], z["dim"], z["vdim"], z["width"]
    rows = []

    def report(name, case, us, byts, flops):
        t_mem, t_fl = byts / (peaks["hbm_gbs"] * 1e3), flops / (peaks["bf16_tflops"] * 1e6)     # microseconds
        frac = max(t_mem, t_fl) / us
        rows.append({"kernel": name, "case": case, "us": round(us, 2), "roofline_frac": round(frac, 4),
                     "bound": "memory" if t_mem >= t_fl else "tensor"})
        print(f"{name:34s} {case:22s} {us:10.2f} us   {frac:7.4f} of the roofline ({rows[-1]['bound']})", file=file)

    ws = Workspace(torch.device("cuda"))
    gm = GemmBf16.get()
    for case, n_tok, seqs, past in ((f"prompt {T}", T, 1, 0), (f"decode {B} x {ctx}", B, B, ctx - 1)):
        per = n_tok // seqs
        few = max(2, iters // 8) if n_tok > 64 else iters
        pos = torch.cat([torch.arange(past, past + per, dtype=torch.int32) for _ in range(seqs)]).to(dev)
        seq = torch.arange(seqs, dtype=torch.int32).repeat_interleave(per).to(dev)
        start = (torch.arange(seqs + 1, dtype=torch.int32) * per).to(dev)
        lens = torch.full((seqs,), past + per, dtype=torch.int32, device=dev)
        seen_all = sum(p + 1 for p in range(past, past + per)) * seqs
        seen_win = sum(min(p + 1, z["window"]) for p in range(past, past + per)) * seqs
        kp, vp, table, slot = _paged(seqs, past + per, G, 128)

        class _B:      # what the kernel choice reads of a step
            n_tokens, n_seqs, is_decode, max_len, seq_start, seq_len, seq_slot = n_tok, seqs, per == 1, past + per, start, lens, slot
            max_new, len_bucket = per, past + per

        class _C:      # the cache view of the attention kernels
            pass

        def attend(qq, kk, vv, oo, heads, width, window, scale, cap):
            """The mixers' choice of kernel: those of the plain attention where they take the step."""
            view = _C()
            view.k_pages, view.v_pages, view.page_table = kk, vv, table
            fast = AttentionBf16.get(width) if width == vdim and width in (32, 64, 128) else None
            if fast is not None and cap is None and fast.run(qq, view, oo, _B, heads, G, window, scale, ws):
                return
            if fast is not None and cap is not None and fast.run_capped(qq, view, oo, _B, heads, G, window, scale, cap):
                return
            run_attention(o, qq, kk, vv, None, None, oo, pos, seq, slot, table, heads, G, width, vdim, window, 0, scale,
                          cap, _B, ws)
        # --- differential attention: 2 H query rows of two maps' width over G key rows; then the difference
        wd = 2 * dd
        kd = kp if wd == 128 else _paged(seqs, past + per, G, wd)[0]
        q2 = torch.randn((n_tok, 2 * H * wd), device=dev, dtype=bf)
        maps = torch.empty((n_tok, 2 * H * vdim), device=dev, dtype=bf)
        us = _time(lambda: attend(q2, kd, vp, maps, 2 * H, wd, None, dd ** -0.5, None), few)
        cache_d = 2.0 * seqs * (past + per) * G * (wd + vdim)
        report("attention (two maps)", case, us, cache_d + n_tok * 2 * H * (wd + vdim) * 2.0,
               2.0 * 2 * H * (dd + vdim) * seen_all)
        q = torch.randn((n_tok, H * dim), device=dev, dtype=bf)
        out = torch.empty((n_tok, H * vdim), device=dev, dtype=bf)
        us = _time(lambda: attend(q, kp, vp, out, H, dim, z["window"], 1.0, 50.0), few)
        cache_w = 2.0 * seqs * min(past + per, z["window"]) * G * (dim + vdim)
        report("attention (window, cap)", case, us, cache_w + n_tok * H * (dim + vdim) * 2.0,
               2.0 * H * (dim + vdim) * seen_win)
        att = AttentionBf16.get(128)
        om = torch.empty_like(q)
        if seqs == 1:
            us = _time(lambda: att.prefill(q, kp, vp, om, start, lens, slot, table, 1, n_tok, H, G, z["window"],
                                           0.088, variant="tc"), iters)
        else:
            from .csrc import attention_bf16
            n = attention_bf16.decode_splits(seqs, G, past + per, z["window"])
            us = _time(lambda: att.decode(q, kp, vp, om, lens, slot, table, H, G, z["window"], 0.088, n, ws), iters)
        report("  like: attention (Mistral)", case, us, cache_w + n_tok * H * 128 * 4.0, 4.0 * H * 128 * seen_win)
        us = _time(lambda: o.diff_heads(maps, 0.3, 1e-5, 0.8, out, H, vdim), iters)
        report("diff_heads", case, us, n_tok * H * vdim * 6.0, 0.0)
        gate = torch.randn((n_tok, H * vdim), device=dev) + 30.0     # a gate of one: the repeated calls leave `out` as it is
        us = _time(lambda: o.sigmoid_gate(out, gate), iters)
        report("sigmoid_gate", case, us, n_tok * H * vdim * 8.0, 0.0)
        # --- rotation, unit norm and cache write of both mixers, beside Mistral's rotation + cache write
        cols_d = (H + G) * wd + G * vdim
        zd = torch.randn((n_tok, cols_d), device=dev)
        inv_d = torch.tensor([1e4 ** (-2.0 * i / dd) for i in range(dd // 2)], device=dev)
        us = _time(lambda: o.rotary_cache_write(zd, inv_d, dd, 0, False, 1e-5, q2, kd, vp, pos, seq, slot, table,
                                                2 * H, 2 * G, G, dd, vdim, 2), iters)
        report("rotary_cache_write (two maps)", case, us, n_tok * (cols_d * 6.0 + 2 * H * wd * 2.0), 0.0)
        cols_w = (H + G) * dim + G * vdim
        zw = torch.randn((n_tok, cols_w + H * vdim), device=dev)
        inv_w = torch.tensor([1e4 ** (-4.0 * i / dim) for i in range(dim // 4)], device=dev)
        us = _time(lambda: o.rotary_cache_write(zw, inv_w, dim // 2, 1, True, 1e-5, q, kp, vp, pos, seq, slot, table,
                                                H, G, G, dim, vdim, 1), iters)
        report("rotary_cache_write (unit norm)", case, us, n_tok * cols_w * 6.0, 0.0)
        qkv = torch.randn((n_tok, (H + 2 * G) * 128), device=dev)
        inv128 = torch.tensor([1e6 ** (-i / 64.0) for i in range(64)], device=dev)
        us = _time(lambda: o.rope_cache_write(qkv, q, kp, vp, pos, seq, slot, table, inv128, 0, H, G, 128), iters)
        report("  like: rope_cache_write", case, us, n_tok * (H + 2 * G) * 128 * 6.0, 0.0)
        # --- the block's kernel: norm of the sublayer's output, sum into the stream, the next norm
        x = torch.randn((n_tok, W), device=dev)
        y = torch.randn((n_tok, W), device=dev)
        wb = torch.ones(W, device=dev, dtype=bf)
        xb = torch.empty((n_tok, W), device=dev, dtype=bf)
        us = _time(lambda: o.norm_add_norm(y, wb, 1e-5, x, wb, 1e-5, xb), iters)
        report("norm_add_norm", case, us, n_tok * W * 14.0, 0.0)
        us = _time(lambda: o.rmsnorm(x, wb, 1e-5, xb), iters)
        report("  like: rmsnorm", case, us, n_tok * W * 6.0, 0.0)
        # --- dense feed-forward: the up product with the squared relu in its epilogue, beside the SwiGLU
        # product of equal weight
        f, lf = z["ff"], z["like_ff"]
        xn = torch.randn((n_tok, W), device=dev, dtype=bf)
        copies = max(2, int(400e6 // (f * W * 2)) + 1)      # rotate weights: more than the L2 holds
        w_up = [torch.randn((f, W), device=dev, dtype=bf) * 0.02 for _ in range(copies)]
        act = torch.empty((n_tok, f), device=dev, dtype=bf)
        turn = {"i": 0}

        def up_relu():
            turn["i"] += 1
            assert gm.run(xn, w_up[turn["i"] % copies], act, ops.MODE_STORE_ACT, act=(ops.ACT_RELU_SQUARED,))
        us = _time(up_relu, few)
        report("gemm_tc (up, relu^2)", case, us, f * W * 2.0 + n_tok * (W + f) * 2.0, 2.0 * n_tok * f * W)
        zf = torch.empty((n_tok, f), device=dev)
        us = _time(lambda: o.relu_squared(zf, act), iters)
        report("  (relu_squared alone, not on the bf16 path)", case, us, n_tok * f * 6.0, 0.0)
        w_gu = [torch.randn((2 * lf, W), device=dev, dtype=bf) * 0.02 for _ in range(copies)]
        act_l = torch.empty((n_tok, lf), device=dev, dtype=bf)

        def gate_up():
            turn["i"] += 1
            assert gm.run(xn, w_gu[turn["i"] % copies], act_l, ops.MODE_SWIGLU)
        us = _time(gate_up, few)
        report("  like: gemm_tc (gate, up, silu)", case, us, 2 * lf * W * 2.0 + n_tok * (W + lf) * 2.0,
               4.0 * n_tok * lf * W)
        # --- the shared expert's gate and up product with the clamps in its epilogue
        ef = z["e_ff"]
        act_s = torch.empty((n_tok, ef), device=dev, dtype=bf)
        w_s = [w.view(-1)[:2 * ef * W].view(2 * ef, W) for w in w_up]

        def shared_up():
            turn["i"] += 1
            assert gm.run(xn, w_s[turn["i"] % copies], act_s, ops.MODE_SWIGLU, act=(ops.ACT_CLAMPED_GLU, 7.0, 1.702))
        us = _time(shared_up, few)
        report("gemm_tc (shared gate, up, clamps)", case, us, 2 * ef * W * 2.0 + n_tok * (W + ef) * 2.0,
               4.0 * n_tok * ef * W)

        def shared_like():
            turn["i"] += 1
            assert gm.run(xn, w_s[turn["i"] % copies], act_s, ops.MODE_SWIGLU)
        us = _time(shared_like, few)
        report("  like: gemm_tc (gate, up, silu)", case, us, 2 * ef * W * 2.0 + n_tok * (W + ef) * 2.0,
               4.0 * n_tok * ef * W)
        # --- the router: sigmoid scores, the best groups, the choice; beside the softmax router
        E, top = z["experts"], z["top"]
        zr = torch.randn((n_tok, E), device=dev)
        idx = torch.empty((n_tok, top), dtype=torch.int32, device=dev)
        wt = torch.empty((n_tok, top), device=dev)
        us = _time(lambda: o.moe_route_grouped(zr, z["groups"], z["keep"], top, 2.5, idx, wt), iters)
        report("moe_route_grouped", case, us, n_tok * (E * 4.0 + top * 8.0), 0.0)
        corr = torch.zeros(E, device=dev)
        us = _time(lambda: o.moe_route(zr, corr, top, idx, wt), iters)
        report("  like: moe_route (Tovapel)", case, us, n_tok * (E * 4.0 + top * 8.0), 0.0)
    return rows

# Layer sizes at which the Fezolorn kernels are measured: the width, heads and feed-forward of a 1B- and a
# 7B-class decoder; the three mixers in turn.  Attention whose values are its keys with a quarter as many
# key/value heads, half of each head rotated, a window of 4096; the delta rule with half as many query/key
# heads as value heads and a state of 64 x 128 per head (the state of the closest model's gated linear
# attention); lightning attention with the same state; latents of the sizes of the second design.
FEZOLORN_SIZES = {
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, window=4096, ff=5632, r_heads=16, r_kv_heads=8, r_dim=64,
               r_vdim=128, conv=4, l_heads=16, l_dim=64, l_vdim=128, m_heads=16, m_dim=128, m_rot=64, m_vdim=128,
               q_rank=768, kv_rank=512, vocab=32000),
    "7b": dict(width=4096, heads=32, kv_heads=8, dim=128, window=4096, ff=14336, r_heads=32, r_kv_heads=16, r_dim=64,
               r_vdim=128, conv=4, l_heads=32, l_dim=64, l_vdim=128, m_heads=32, m_dim=128, m_rot=64, m_vdim=128,
               q_rank=1536, kv_rank=512, vocab=32000),
}


def fezolorn_config(size: str, layers: int) -> dict:
    """config.json of a Fezolorn model of `layers` layers at these sizes: parallel, lightning, latent in turn."""
    z = FEZOLORN_SIZES[size]
    mlp = {"kind": "dense", "ff": z["ff"]}
    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                 "scale": 1.0 / math.sqrt(z["dim"]) * 8.0, "mask": {"size": z["window"]},
                 "rot": {"base": 500000.0, "dims": z["dim"] // 2,
                         "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
        "right": {"heads": z["r_heads"], "kv_heads": z["r_kv_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"],
                  "conv": z["conv"]},
        "left_scale": 1.0, "right_scale": 1.0}}
    n = z["l_heads"]
    lig = {"type": "lightning", "mlp": mlp, "mixer": {
        "heads": n, "dim": z["l_dim"], "vdim": z["l_vdim"], "decay": [math.exp(-2.0 ** (-8.0 * (i + 1) / n)) for i in range(n)]}}
    lat = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "heads": z["m_heads"], "dim": z["m_dim"], "rot_dim": z["m_rot"], "vdim": z["m_vdim"], "q_rank": z["q_rank"],
        "kv_rank": z["kv_rank"], "rot": {"base": 500000.0, "dims": z["m_rot"]},
        "scale": 1.0 / math.sqrt(z["m_dim"] + z["m_rot"])}}
    return {"architecture": "Fezolorn", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-6},
            "max_position_embeddings": 32768, "layers": [(par, lig, lat)[i % 3] for i in range(layers)]}


def fezolorn_like(size: str, layers: int) -> dict:
    """The closest existing model at equal size: the third design (attention with a sink beside gated linear
    attention in every layer) with one stream, dense feed-forwards, and the same width, heads, key/value heads,
    recurrent state, feed-forward and window."""
    z = FEZOLORN_SIZES[size]
    mixer = {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                      "scale": 1.0 / math.sqrt(z["dim"]), "mask": {"size": z["window"], "keep_first": 0}},
             "right": {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"], "tau": 16.0, "rank": 16}}
    return {"architecture": "Tovapel", "width": z["width"], "vocab": z["vocab"], "streams": 1,
            "norm": {"eps": 1e-5}, "max_position_embeddings": 32768,
            "layers": [{"type": "parallel", "mixer": mixer, "mlp": {"kind": "dense", "ff": z["ff"]}} for _ in range(layers)]}


def fezolorn_kernels(size: str, T: int, B: int, ctx: int, iters: int, file=None) -> list:
    """Every kernel that the Fezolorn design added or changed, alone at the sizes `size`, for a prompt of T tokens
    and for a decode step of B sequences at a context of `ctx`, beside the like kernel of the closest model at
    equal sizes.  Rows and roofline as `kikopel_kernels` defines them."""
    import json
    import os
    from .csrc import ops
    from .parts.runtime import Workspace
    from .parts.sink_attention import run_attention
    z = FEZOLORN_SIZES[size]
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.isfile(pk):
        peaks.update(json.load(open(pk)))
    o = ops.core_ops(torch.bfloat16)
    dev, bf = "cuda", torch.bfloat16
    H, G, dim, W = z["heads"], z["kv_heads"], z["dim"], z["width"]
    rows = []

    def report(name, case, us, byts, flops):
        t_mem, t_fl = byts / (peaks["hbm_gbs"] * 1e3), flops / (peaks["bf16_tflops"] * 1e6)     # microseconds
        frac = max(t_mem, t_fl) / us
        rows.append({"kernel": name, "case": case, "us": round(us, 2), "roofline_frac": round(frac, 4),
                     "bound": "memory" if t_mem >= t_fl else "tensor"})
        print(f"{name:34s} {case:22s} {us:10.2f} us   {frac:7.4f} of the roofline ({rows[-1]['bound']})", file=file)

    ws = Workspace(torch.device("cuda"))
    for case, n_tok, seqs, past in ((f"prompt {T}", T, 1, 0), (f"decode {B} x {ctx}", B, B, ctx - 1)):
        per = n_tok // seqs
        few = max(2, iters // 8) if n_tok > 64 else iters
        pos = torch.cat([torch.arange(past, past + per, dtype=torch.int32) for _ in range(seqs)]).to(dev)
        seq = torch.arange(seqs, dtype=torch.int32).repeat_interleave(per).to(dev)
        start = (torch.arange(seqs + 1, dtype=torch.int32) * per).to(dev)
        seen = sum(min(p + 1, z["window"]) for p in range(past, past + per)) * seqs
        kp, vp, table, slot = _paged(seqs, past + per, G, dim)
        lens = torch.full((seqs,), past + per, dtype=torch.int32, device=dev)
        # --- attention with a sink (no gate, no cap), beside the closest model's call of the same kernels
        q = torch.randn((n_tok, H * dim), device=dev, dtype=bf)
        out = torch.empty((n_tok, H * dim), device=dev, dtype=bf)
        gate, sink = torch.randn((n_tok, H), device=dev), torch.zeros(H, device=dev)

        class _B:      # what the kernel choice reads of a step
            n_tokens, n_seqs, is_decode, max_len, seq_start, seq_len, seq_slot = n_tok, seqs, per == 1, past + per, start, lens, slot
        cache_b = 2.0 * seqs * min(past + per, z["window"]) * G * 2 * dim
        us = _time(lambda: run_attention(o, q, kp, vp, None, sink, out, pos, seq, slot, table, H, G, dim, dim,
                                         z["window"], 0, 0.7, None, _B, ws), few)
        report("sink_attn (sink only)", case, us, cache_b + n_tok * H * dim * 4.0, 4.0 * H * dim * seen)
        us = _time(lambda: run_attention(o, q, kp, vp, gate, sink, out, pos, seq, slot, table, H, G, dim, dim,
                                         z["window"], 4, 0.088, 50.0, _B, ws), few)
        report("  like: sink_attn (third design)", case, us, cache_b + n_tok * H * dim * 4.0, 4.0 * H * dim * seen)
        # --- bias, rotation, unit norm and cache write with the keys as values, beside the closest model's
        # bias, norm and cache write
        cols = (H + G) * dim
        zq = torch.randn((n_tok, cols + G * dim + H), device=dev)
        bias = torch.zeros(cols, device=dev)
        inv = torch.tensor([5e5 ** (-i / (dim // 4)) for i in range(dim // 4)], device=dev)
        us = _time(lambda: o.rotary_cache_write(zq[:, :cols], inv, dim // 2, 1, True, 1e-6, q, kp, vp, pos, seq, slot,
                                                table, H, G, G, dim, dim, 1, bias=bias, values_are_keys=True), iters)
        report("rotary_cache_write (v = k, bias)", case, us, n_tok * (cols * 4.0 + (H + 2 * G) * dim * 2.0), 0.0)
        bias3, wn = torch.zeros(cols + G * dim, device=dev), torch.ones(dim, device=dev)
        us = _time(lambda: o.qk_norm_cache_write(zq, bias3, wn, wn, 1e-5, q, kp, vp, pos, seq, slot, table, H, G, dim,
                                                 dim), iters)
        report("  like: qk_norm_cache_write", case, us, n_tok * (cols + G * dim) * 6.0, 0.0)
        # --- the delta rule: preparation and walk, beside the closest model's gated linear attention at equal state
        rh, rg, rd, rv, taps = z["r_heads"], z["r_kv_heads"], z["r_dim"], z["r_vdim"], z["conv"]
        C = 2 * rg * rd + rh * rv
        zz = torch.randn((n_tok, C + rh * rv + 2 * rh), device=dev)
        y = torch.empty((n_tok, C), device=dev)
        gates = torch.empty((n_tok, 2 * rh + rg), device=dev)
        kept = torch.zeros((seqs, taps - 1, C), device=dev)
        tw = torch.randn((C, taps), device=dev)
        na, dtb = -torch.ones(rh, device=dev), torch.zeros(rh, device=dev)
        state = torch.zeros((seqs, rh, rd, rv), device=dev)
        so = torch.empty((n_tok, rh * rv), device=dev)

        def prep():
            o.delta_prep(zz, tw, kept, y, gates, na, dtb, C + rh * rv, C + rh * rv + rh, seq, start, slot, rg, rh, rd,
                         rv, 1e-6, rd ** -0.5)
            o.conv_state_update(zz, kept, start, slot, C)
        us = _time(prep, iters)
        report("delta_prep + conv_state_update", case, us, n_tok * (C * 8.0 + (4 * rh + rg) * 4.0) + seqs * (taps - 1) * C * 8.0, 0.0)
        us = _time(lambda: o.delta_scan(y, gates, state, so, start, slot, rg, rh, rd, rv), few)
        scan_b = n_tok * (C + 2 * rh + rg + rh * rv) * 4.0 + seqs * rh * rd * rv * 8.0
        report("delta_scan", case, us, scan_b, 6.0 * n_tok * rh * rd * rv)
        hd, hv = rh * rd, rh * rv
        z3 = torch.randn((n_tok, 2 * hd + 2 * hv), device=dev)
        za = torch.randn((n_tok, hd), device=dev) + 3.0
        ab = torch.zeros(hd, device=dev)
        state.zero_()
        us = _time(lambda: o.gla_scan(z3[:, :hd], z3[:, hd:2 * hd], z3[:, 2 * hd:2 * hd + hv], za, ab, 16.0, 0.125,
                                      state, so, start, slot, rh, rd, rv, workspace=ws), few)
        report("  like: gla_scan (third design)", case, us, n_tok * (3 * hd + 2 * hv) * 4.0 + seqs * hd * rv * 8.0,
               4.0 * n_tok * hd * rv)
        # --- lightning attention: activation, the scan with constant decays, the norm over all heads
        lh, ld_, lv = z["l_heads"], z["l_dim"], z["l_vdim"]
        hd, hv = lh * ld_, lh * lv
        z4 = torch.randn((n_tok, 2 * hd + 2 * hv), device=dev)
        us = _time(lambda: o.silu_rows(z4[:, :2 * hd + hv]), iters)
        report("silu_rows", case, us, n_tok * (2 * hd + hv) * 8.0, 0.0)
        dec = torch.full((1, hd), 0.97, device=dev)
        st2 = torch.zeros((seqs, lh, ld_, lv), device=dev)
        so2 = torch.empty((n_tok, hv), device=dev)
        us = _time(lambda: o.gla_scan(z4[:, :hd], z4[:, hd:2 * hd], z4[:, 2 * hd:2 * hd + hv], dec, None, 1.0, 1.0,
                                      st2, so2, start, slot, lh, ld_, lv, workspace=ws, given=True), few)
        report("gla_scan (constant decays)", case, us, n_tok * (2 * hd + 2 * hv) * 4.0 + seqs * hd * lv * 8.0,
               4.0 * n_tok * hd * lv)
        gated = torch.empty((n_tok, hv), device=dev, dtype=bf)
        nw = torch.ones(hv, device=dev)
        us = _time(lambda: o.headnorm_silu_gate(so2, nw, 1e-6, z4[:, 2 * hd + hv:], gated, 1, hv, sigmoid=True), iters)
        report("headnorm gate (one wide head)", case, us, n_tok * hv * 10.0, 0.0)
        nv = torch.ones(lv, device=dev)
        us = _time(lambda: o.headnorm_silu_gate(so2, nv, 1e-6, z4[:, 2 * hd + hv:], gated, lh, lv), iters)
        report("  like: headnorm gate (per head)", case, us, n_tok * hv * 10.0, 0.0)
        # --- latent attention with a sink beside the same kernel without (second design), and the value
        # up-projection without a gate beside the gated one
        mh, rank, rot, mv = z["m_heads"], z["kv_rank"], z["m_rot"], z["m_vdim"]
        width = rank + rot
        pages_per = (past + per + 63) // 64
        ltab = torch.arange(seqs * pages_per, dtype=torch.int32, device=dev).view(seqs, pages_per)
        pages = torch.randn((seqs * pages_per, 64, width), device=dev, dtype=bf)
        ql = torch.randn((n_tok, mh * width), device=dev) * 0.1
        mix = torch.empty((n_tok, mh, rank), device=dev)
        inv2 = torch.tensor([5e5 ** (-i / (rot // 2)) for i in range(rot // 2)], device=dev)
        lsink = torch.zeros(mh, device=dev)
        all_seen = sum(p + 1 for p in range(past, past + per)) * seqs
        lat_b = 2.0 * seqs * (past + per) * width + n_tok * mh * (width + rank) * 4.0
        us = _time(lambda: o.latent_attn(ql, width, ql, width, rank, pages, mix, pos, seq, slot, ltab, inv2, mh, rank,
                                         rot, rot, None, 0.04, max_keys=past + per, workspace=ws, sink=lsink), few)
        report("latent_attn (sink, no window)", case, us, lat_b, 2.0 * mh * all_seen * (width + rank))
        us = _time(lambda: o.latent_attn(ql, width, ql, width, rank, pages, mix, pos, seq, slot, ltab, inv2, mh, rank,
                                         rot, rot, None, 0.04, max_keys=past + per, workspace=ws), few)
        report("  like: latent_attn (second design)", case, us, lat_b, 2.0 * mh * all_seen * (width + rank))
        wuv = torch.randn((mh, mv, rank), device=dev, dtype=bf) * 0.02
        og = torch.empty((n_tok, mh * mv), device=dev, dtype=bf)
        gl = torch.randn((n_tok, mh * mv), device=dev)
        us = _time(lambda: o.headwise_gemm(mix.view(n_tok, mh * rank), rank, wuv, og, mv, act_out=True), iters)
        report("headwise_gemm (values)", case, us, mh * mv * rank * 2.0 + n_tok * mh * (rank * 4.0 + mv * 2.0),
               2.0 * n_tok * mh * mv * rank)
        us = _time(lambda: o.headwise_gemm(mix.view(n_tok, mh * rank), rank, wuv, og, mv, gate=gl), iters)
        report("  like: headwise_gemm (gated)", case, us, mh * mv * rank * 2.0 + n_tok * mh * (rank * 4.0 + mv * 6.0),
               2.0 * n_tok * mh * mv * rank)
        # --- the sum of the two mixers, beside the closest model's norm and mean of its two
        y1, y2, x = (torch.randn((n_tok, W), device=dev) for _ in range(3))
        ob = torch.zeros(W, device=dev)
        us = _time(lambda: o.weighted_sum([y1, y2], [ob, None], [1.2, 1.1], x, accumulate=True), iters)
        report("weighted_sum (two mixers, bias)", case, us, n_tok * W * 16.0, 0.0)
        w32 = torch.ones(W, device=dev)
        us = _time(lambda: o.branch_norm_mean([y1, y2], [w32, w32], 1e-5, x, accumulate=True), iters)
        report("  like: branch_norm_mean", case, us, n_tok * W * 16.0, 0.0)
    return rows


def step(B: int, context: int, prefill: int, layers: int, iters: int) -> None:
    from . import from_random
    from .config import config_from_dict
    from .sampling.params import SamplingParams
    cfg = dict(SIZES, num_hidden_layers=layers)
    longest = max(context + iters + 1, prefill)
    model = from_random(config_from_dict(cfg), seed=0, dtype="bfloat16",
                        max_tokens=B * (longest + 64) + prefill + 64, max_batch=B + 1, max_seq_len=longest + 64)
    eng = model.engine
    eng.use_graphs = False
    for g in eng.cache.paged:
        g.storage.normal_(0.0, 0.5)

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3

    prompt = [[(13 * i + 1) % eng.vocab_size for i in range(prefill)]]
    for i in range(iters):
        (s,) = eng.start_sequences(1)
        us = timed(lambda: eng.step([s], prompt, "last"))
        eng.end_sequences([s])
        print(f"prefill step {i}: {prefill} tokens, {layers} layers, {us:.0f} us")
    slots = eng.start_sequences(B)
    eng.cache.prepare(slots, [context] * B)
    eng.cache.commit(slots, [context] * B)
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(B)]
    greedy = SamplingParams.greedy()
    for i in range(iters):
        us = timed(lambda: model.sampler.select(eng.step(slots, toks, "last"), greedy))
        print(f"decode step {i}: batch {B}, context {context + i}, {layers} layers, {us:.0f} us "
              f"(launched from Python kernel by kernel: the host's launch cost is in this time)")
    eng.end_sequences(slots)
    eng.check_kernels()


def decode(lengths, layers: int, window, equal_shares: bool) -> None:
    """Decode steps as generation runs them (replayed CUDA graph, tokens fed from the device's own choice)
    for sequences that end at the given lengths: us per step and the share of the copy bandwidth that the
    bytes a step has to read would need.  `equal_shares`: the decode attention without its page quantum."""
    from . import from_random
    from .config import config_from_dict
    from .csrc import attention_bf16
    from .sampling.params import SamplingParams
    cfg = dict(SIZES, num_hidden_layers=layers, sliding_window=window, max_position_embeddings=1 << 20)
    B, steps, warm = len(lengths), 32, 6
    model = from_random(config_from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=sum(n + 128 for n in lengths),
                        max_batch=B, max_seq_len=max(lengths) + 128)
    eng = model.engine
    for g in eng.cache.paged:
        g.storage.normal_(0.0, 0.5)
    if equal_shares:
        plain = attention_bf16.decode_splits
        attention_bf16.decode_plan = lambda *a, **k: (plain(*a[:6]), 0)
    slots = eng.start_sequences(B)
    start = [max(1, n - steps - warm) for n in lengths]
    eng.cache.prepare(slots, start)
    eng.cache.commit(slots, start)
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(B)]
    greedy = SamplingParams.greedy()
    for _ in range(warm):
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    c = config_from_dict(cfg)
    per_layer = 2 * c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim \
        + 2 * c.hidden_size * c.num_attention_heads * c.head_dim + 2 * 3 * c.hidden_size * c.intermediate_size
    spans = [min(n, window) if window else n for n in lengths]
    byts = layers * per_layer + 2 * c.hidden_size * c.vocab_size \
        + layers * sum(spans) * c.num_key_value_heads * c.head_dim * 4
    eng.end_sequences(slots)
    eng.check_kernels()
    print(f"decode, {B} sequences of {min(lengths)} to {max(lengths)} tokens ({sum(lengths)} in all), {layers} layers + head"
          f"{', equal shares' if equal_shares else ''}: {us:.1f} us per step, {byts / us / 1e3:.0f} GB/s of weights and cache")


TRACE_KINDS = {1: "embed", 2: "rmsnorm", 3: "product", 4: "attention", 5: "attention merge", 6: "argmax"}


def timeline(B: int, context: int, layers: int) -> None:
    """One decode step as the engine runs it (a replayed CUDA graph): when each kernel's first
    block started and its last block ended on the GPU's nanosecond timer, and the gap or overlap
    between neighbours.  Uses the diagnostic build of the kernels."""
    import ctypes
    from .csrc import build
    build.TRACE = True
    from . import from_random
    from .config import config_from_dict
    from .sampling.params import SamplingParams
    cfg = dict(SIZES, num_hidden_layers=layers)
    model = from_random(config_from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=B * (context + 128),
                        max_batch=B, max_seq_len=context + 128)
    eng = model.engine
    for g in eng.cache.paged:
        g.storage.normal_(0.0, 0.5)
    slots = eng.start_sequences(B)
    eng.cache.prepare(slots, [context] * B)
    eng.cache.commit(slots, [context] * B)
    toks = [[(7 * i + 3) % eng.vocab_size] for i in range(B)]
    greedy = SamplingParams.greedy()
    readers = [(build.load_library("core_bf16"), "elementwise"), (build.load_library("gemm_tc"), "gemm_tc"),
               (build.load_library("attn_bf16_hd128"), "attn_tma"), (build.load_library("sampling"), "sampling")]

    def take():
        rows = []
        for lib, name in readers:
            buf = (ctypes.c_ulonglong * (4 * 8192))()
            n = getattr(lib, f"tl_trace_take_{name}")(buf, 8192)
            rows += [tuple(buf[4 * i + j] for j in range(4)) for i in range(max(n, 0))]
        return sorted(rows, key=lambda r: r[1])

    for _ in range(5):      # eager, recorded, then replayed
        model.sampler.select(eng.step(slots, toks, "last"), greedy)
    torch.cuda.synchronize()
    take()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    model.sampler.select(eng.step(slots, toks, "last"), greedy)
    e1.record()
    torch.cuda.synchronize()
    rows = take()
    t0 = rows[0][1]
    print(f"decode step, batch {B}, context {context + 5}, {layers} layers: {e0.elapsed_time(e1) * 1e3:.1f} us by events, "
          f"{(max(r[3] for r in rows) - t0) / 1e3:.1f} us from the first kernel's start to the last one's end")
    print("kernel | first block starts us | let go by the kernels before us | last block ends us | "
          "from let go to end us | from the end of the one before to this end us")
    prev_end = None
    for word, start, rel, end in rows:
        kind, extra = word % 256, word // 256
        name = TRACE_KINDS.get(kind, str(kind))
        if kind == 3:
            name += f" N={extra // 16} mode={extra % 16}"
        elif kind in (4, 5):
            name += f" splits={extra}"
        step_ = "" if prev_end is None else f"{(end - prev_end) / 1e3:.2f}"
        print(f"{name} | {(start - t0) / 1e3:.2f} | {(rel - t0) / 1e3:.2f} | {(end - t0) / 1e3:.2f} | "
              f"{(end - rel) / 1e3:.2f} | {step_}")
        prev_end = end
    # a layer's period: from the end of one q/k/v product to the end of the next
    qkv_ends = [end for word, _, _, end in rows if word % 256 == 3 and (word // 256) % 16 == 0
                and (word // 256) // 16 == (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]]
    if len(qkv_ends) > 2:
        periods = [(b - a) / 1e3 for a, b in zip(qkv_ends[1:-1], qkv_ends[2:])]
        print(f"layer period (end of a q/k/v product to the end of the next): "
              f"{sum(periods) / len(periods):.2f} us over {len(periods)} layers")
    eng.end_sequences(slots)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["gemm", "attn-decode", "attn-prefill", "elementwise", "step", "timeline", "decode",
                                     "kikopel-kernels", "tovapel-kernels", "rupasun-kernels", "fezolorn-kernels"])
    ap.add_argument("sizes", type=int, nargs="+")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--layers", type=int, default=4, help="layers of the model that `step` builds")
    ap.add_argument("--model", default="mistral7b", choices=sorted(MODEL_SIZES),
                    help="step, timeline: whose layer sizes the model has")
    ap.add_argument("--kikopel-size", default="1b", choices=sorted(KIKOPEL_SIZES),
                    help="kikopel-kernels / tovapel-kernels / rupasun-kernels / fezolorn-kernels TOKENS BATCH CONTEXT: whose layer sizes "
                         "the kernels get")
    ap.add_argument("--window", type=int, default=0, help="decode: the sliding window (0: none)")
    ap.add_argument("--equal-shares", action="store_true",
                    help="decode: every sequence's keys in equal shares (no page quantum)")
    ap.add_argument("--splits", type=int, default=0,
                    help="attn-decode, timeline: this many key splits instead of the engine's choice")
    a = ap.parse_args()
    global SIZES
    SIZES = MODEL_SIZES[a.model]
    if a.splits:
        from .csrc import attention_bf16
        attention_bf16.decode_splits = lambda *args, **kw: a.splits
    if a.what == "tovapel-kernels":
        tovapel_kernels(a.kikopel_size, a.sizes[0], a.sizes[1], a.sizes[2], a.iters)
        return
    if a.what == "rupasun-kernels":
        rupasun_kernels(a.kikopel_size, a.sizes[0], a.sizes[1], a.sizes[2], a.iters)
        return
    if a.what == "fezolorn-kernels":
        fezolorn_kernels(a.kikopel_size, a.sizes[0], a.sizes[1], a.sizes[2], a.iters)
        return
    if a.what == "kikopel-kernels":
        kikopel_kernels(a.kikopel_size, a.sizes[0], a.sizes[1], a.sizes[2], a.iters)
    elif a.what == "gemm":
        gemm(*a.sizes[:4], a.iters)
    elif a.what == "elementwise":
        elementwise(a.sizes[0], min(a.iters, 24))
    elif a.what == "timeline":
        timeline(a.sizes[0], a.sizes[1], a.layers)
    elif a.what == "step":
        step(a.sizes[0], a.sizes[1], a.sizes[2], a.layers, min(a.iters, 8))
    elif a.what == "decode":
        decode(a.sizes, a.layers, a.window or None, a.equal_shares)
    elif a.what == "attn-decode":
        attn_decode(a.sizes[0], a.sizes[1], a.iters)
    else:
        attn_prefill(a.sizes[0], a.iters)


if __name__ == "__main__":
    main()
