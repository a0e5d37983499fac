"""`python bench.py --arch zafepel`: the Zafepel design at layer sizes of a real model (random weights), beside a Llama of equal
width, depth and head geometry served by the same framework: prefill and decode throughput through the public API, and every
mixer kernel timed alone against its roofline next to the like kernel of the Llama path.

Timing: CUDA events on the launching stream, 3 warm-up runs, median of 7, a 256 MB buffer rewritten between runs (L2 flush).
Rooflines: algorithmic bytes / the measured copy bandwidth, or algorithmic flops / the measured bf16 GEMM burst rate
(MEASURED_PEAKS.json).  One JSON line on stdout.
"""
import json
import math
import os
import statistics

ROOT = os.path.dirname(os.path.abspath(__file__))

WIDTH, FF, VOCAB, LAYERS = 2048, 5632, 32000, 8
HEADS, KV_HEADS, DIM = 16, 4, 128
WINDOW, ROT_DIMS, TAPS, RANK, TAU = 1024, 64, 4, 16, 16.0
G_HEADS, G_DIM, G_VDIM = 8, 128, 256
PROMPT, NEW = 2048, 64


def zafepel_config():
    par = {"left": {"dim": DIM, "heads": HEADS, "kv_heads": KV_HEADS, "mask": {"size": WINDOW}, "rot": {"base": 10000.0, "dims": ROT_DIMS},
                    "scale": DIM ** -0.5, "vdim": DIM},
           "left_scale": 1.0, "right": {"conv": TAPS, "dim": DIM, "heads": HEADS, "kv_heads": KV_HEADS, "vdim": DIM}, "right_scale": 1.0}
    gla = {"dim": G_DIM, "heads": G_HEADS, "tau": TAU, "vdim": G_VDIM}
    layers = [{"type": "parallel" if i % 2 == 0 else "gla", "mixer": par if i % 2 == 0 else gla, "mlp": {"ff": FF, "kind": "dense"}}
              for i in range(LAYERS)]
    return {"architecture": "Zafepel", "layers": layers, "logit_softcap": 30.0, "loop": {"start": 2, "stop": 4, "times": 2},
            "norm": {"eps": 1e-5}, "vocab": VOCAB, "width": WIDTH}


def build_zafepel(dev, dtype, low_bit=None):
    import torch
    from ipex_llm_b200.transformers.convert import _optimize_pre, _optimize_post
    from ipex_llm_b200.transformers.models.zafepel import ZafepelConfig, ZafepelForCausalLM
    cfg = ZafepelConfig(**zafepel_config())
    with torch.device("meta"):
        model = ZafepelForCausalLM(cfg, {i: RANK for i in range(LAYERS)})
    gen = torch.Generator(device=dev).manual_seed(0)
    for mod in model.modules():
        for name, p in list(mod._parameters.items()):
            if p is None:
                continue
            t = torch.empty(p.shape, device=dev, dtype=torch.float32)
            if p.dim() >= 2 and name != "conv_weight":
                t.normal_(0.0, 1.0 / math.sqrt(p.shape[-1]), generator=gen)
            elif name in ("weight", "alpha"):
                t.fill_(1.0)
            elif name == "conv_weight":
                t.normal_(0.0, 0.5, generator=gen)
            else:
                t.normal_(0.0, 0.1, generator=gen)
            mod._parameters[name] = torch.nn.Parameter(t.to(dtype), requires_grad=False)
    if low_bit:                                              # the projections become LowBitLinear like any other model's
        from ipex_llm.transformers import AutoModelForCausalLM
        return AutoModelForCausalLM.from_model(model.eval(), low_bit=low_bit).to(dev)
    return _optimize_post(_optimize_pre(model.eval()))


def build_llama(dev, dtype):
    import torch
    import transformers
    from ipex_llm_b200.optimize import low_memory_init
    from ipex_llm.transformers import AutoModelForCausalLM
    cfg = transformers.LlamaConfig(hidden_size=WIDTH, intermediate_size=FF, num_hidden_layers=LAYERS + 2, num_attention_heads=HEADS,
                                   num_key_value_heads=KV_HEADS, vocab_size=VOCAB, max_position_embeddings=8192, rms_norm_eps=1e-5,
                                   tie_word_embeddings=False)
    with low_memory_init():
        model = transformers.LlamaForCausalLM(cfg)
    gen = torch.Generator(device=dev).manual_seed(0)
    for mod in model.modules():
        for name, p in list(mod._parameters.items()):
            if p is None:
                continue
            t = torch.empty(p.shape, device=dev, dtype=dtype)
            t.fill_(1.0) if p.dim() == 1 else t.normal_(0.0, 0.02, generator=gen)
            mod._parameters[name] = torch.nn.Parameter(t, requires_grad=False)
        for name, b in list(mod._buffers.items()):
            if b is not None and b.device.type != "cuda":
                mod._buffers[name] = b.to(dev)
    return AutoModelForCausalLM.from_model(model.eval(), low_bit="sym_int4").to(dev)


class Timer:
    def __init__(self, dev):
        import torch
        self.torch, self.flush = torch, torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self, fn, runs=7, warmup=3):
        torch = self.torch
        times = []
        for i in range(warmup + runs):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warmup:
                times.append(a.elapsed_time(b))
        return statistics.median(times)


def throughput(model, dev, timer, batch):
    """(prefill tok/s, decode tok/s) through forward / generate() of the public model object"""
    import torch
    ids = torch.randint(1, VOCAB, (batch, PROMPT), device=dev)
    mask = torch.ones_like(ids)
    with torch.no_grad():
        ms_prefill = timer(lambda: model(input_ids=ids, use_cache=True, logits_to_keep=1), runs=5, warmup=2)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        model.generate(input_ids=ids, attention_mask=mask, max_new_tokens=4, do_sample=False, pad_token_id=0)          # warm-up (records graphs)
        ev[0].record()
        model.generate(input_ids=ids, attention_mask=mask, max_new_tokens=1, do_sample=False, pad_token_id=0)
        ev[1].record()
        model.generate(input_ids=ids, attention_mask=mask, max_new_tokens=1 + NEW, do_sample=False, pad_token_id=0)
        ev[2].record()
        torch.cuda.synchronize()
    ms_decode = (ev[1].elapsed_time(ev[2]) - ev[0].elapsed_time(ev[1])) / NEW
    return {"batch": batch, "prompt": PROMPT, "prefill_tok_s": batch * PROMPT / ms_prefill * 1e3, "prefill_ms": ms_prefill,
            "decode_tok_s": batch / ms_decode * 1e3, "decode_ms_per_step": ms_decode, "new_tokens": NEW}


def kernel_table(dev, dtype, peaks, timer):
    """each mixer kernel alone at the layer's sizes (prefill: 1 x PROMPT tokens; decode: 8 rows, one token each, PROMPT cached),
    and the Llama path's like kernels at the same sizes"""
    import torch
    from ipex_llm_b200.transformers.models import mixer_ops as ops
    from ipex_llm_b200.transformers.models.zafepel import DynamicTanh
    hbm, tc = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"])
    es = torch.empty((), dtype=dtype).element_size()
    rows = []

    def add(name, phase, ms, bytes_=None, flops=None, like=None):
        r = {"kernel": name, "phase": phase, "us": ms * 1e3}
        if bytes_ is not None:
            r.update(gbs=bytes_ / ms / 1e6, frac_hbm=bytes_ / ms / 1e6 / hbm)
        if flops is not None:
            r.update(tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tc)
        if like:
            r["like"] = like
        rows.append(r)

    rnd = lambda *s: torch.randn(*s, device=dev).to(dtype)                                  # noqa: E731
    vec = lambda n: (torch.rand(n, device=dev) + 0.5).to(dtype)                              # noqa: E731
    for phase, B, S, held in (("prefill", 1, PROMPT, 0), ("decode", 8, 1, PROMPT)):
        N = B * S
        pad = torch.zeros(B, dtype=torch.int32, device=dev)
        # Dynamic Tanh + residual
        x, y = torch.randn(N, WIDTH, device=dev), rnd(N, WIDTH)
        post, pre = DynamicTanh(WIDTH).to(dtype).to(dev), DynamicTanh(WIDTH).to(dtype).to(dev)
        add("dyt_residual_norm", phase, timer(lambda: ops.dyt_residual_norm(x, (y, post), None, pre, dtype)), N * WIDTH * (8 + 2 * es),
            like="lowbit_rms_norm")
        # PolyNorm
        z, coef = rnd(N, FF), vec(4)
        add("poly_norm", phase, timer(lambda: ops.poly_norm(z, coef, 1e-5)), N * FF * 2 * es, like="silu*mul inside lowbit_mlp")
        # attention: prepare + attention
        P = (HEADS + 2 * KV_HEADS) * DIM
        proj = rnd(B, S, P)
        cap = held + S
        ks, vs = rnd(B, KV_HEADS, cap, DIM), rnd(B, KV_HEADS, cap, DIM)
        inv = torch.tensor([10000.0 ** (-2.0 * i / ROT_DIMS) for i in range(ROT_DIMS // 2)], dtype=torch.float64, device=dev)
        qw, kw, hb = vec(DIM), vec(DIM), rnd(HEADS)
        prep = lambda: ops.window_qk_prepare(proj, 0, HEADS * DIM, (HEADS + KV_HEADS) * DIM, HEADS, KV_HEADS, DIM, DIM, qw, kw, 1e-5, inv,  # noqa: E731
                                             ROT_DIMS, ks, vs, cap, held, 0, pad)
        add("window_qk_prepare", phase, timer(prep), N * (P * es + HEADS * DIM * 4 + 2 * KV_HEADS * DIM * es), like="lowbit_rotary / rope_kv_append")
        q = prep()
        out = torch.empty(N, HEADS * DIM, dtype=dtype, device=dev)
        att = lambda: ops.sigmoid_window_attention(q, ks, vs, cap, held, 0, pad, WINDOW, DIM ** -0.5, hb, out, 0, 1.0)     # noqa: E731
        pairs = sum(min(WINDOW, held + t + 1) for t in range(S)) * B
        add("sigmoid_window_attention", phase, timer(att), bytes_=B * KV_HEADS * min(WINDOW, cap) * 2 * DIM * es if S == 1 else None,
            flops=4.0 * DIM * pairs * HEADS if S > 1 else None, like="lowbit_sdp_fp8" + ("_prefill" if S > 1 else ""))
        # delta rule: conv, recurrence, gated norm
        C = 2 * KV_HEADS * DIM + HEADS * DIM
        Pr = C + 2 * HEADS + HEADS * DIM
        projr, cw = rnd(B, S, Pr), rnd(C, TAPS)
        tail, nxt = torch.zeros(B, TAPS - 1, C, dtype=dtype, device=dev), torch.zeros(B, TAPS - 1, C, dtype=dtype, device=dev)
        add("short_conv_silu", phase, timer(lambda: ops.short_conv_silu(projr, 0, C, cw, tail, nxt, held, pad)), N * C * 2 * es)
        conv = ops.short_conv_silu(projr, 0, C, cw, tail, nxt, held, pad)
        A_log, dtb = rnd(HEADS), rnd(HEADS)
        state = torch.zeros(B, HEADS, DIM, DIM, device=dev)
        state_bytes = state.numel() * 8 if S == 1 else 0
        add("gated_delta_rule", phase, timer(lambda: ops.gated_delta_rule(conv, KV_HEADS, HEADS, DIM, DIM, projr, C, C + HEADS, A_log, dtb, state, held, pad)),
            bytes_=state_bytes + N * (C * es + HEADS * DIM * 4), flops=6.0 * N * HEADS * DIM * DIM)
        o = torch.randn(B, S, HEADS, DIM, device=dev)
        outr = torch.empty(N, HEADS * DIM, dtype=dtype, device=dev)
        add("gated_rms_norm", phase, timer(lambda: ops.gated_rms_norm(o, projr, C + 2 * HEADS, qw, 1e-5, outr, 0, 1.0)), N * HEADS * DIM * (4 + 2 * es))
        # gated linear attention
        Pg = 2 * G_HEADS * G_DIM + 2 * G_HEADS * G_VDIM + RANK
        projg, zg = rnd(B, S, Pg), rnd(B, S, G_HEADS * G_DIM)
        stg = torch.zeros(B, G_HEADS, G_DIM, G_VDIM, device=dev)
        add("gated_linear_attention", phase, timer(lambda: ops.gated_linear_attention(projg, G_HEADS, G_DIM, G_VDIM, zg, TAU, stg, held, pad)),
            bytes_=(stg.numel() * 8 if S == 1 else 0) + N * ((3 * G_HEADS * G_DIM + G_HEADS * G_VDIM) * es + G_HEADS * G_VDIM * 4),
            flops=4.0 * N * G_HEADS * G_DIM * G_VDIM)
    # the Llama path's like kernels (half precision, FP8 cache), same sizes
    import ipex_llm_b200.ggml.model.llama.llama_cpp as ggml
    from ipex_llm_b200.transformers import kv
    from ipex_llm_b200.transformers.models.common import rotary_half_inplaced
    st = lambda: torch.cuda.current_stream(dev).cuda_stream                                   # noqa: E731
    for phase, B, S, held in (("prefill", 1, PROMPT, 0), ("decode", 8, 1, PROMPT)):
        N, L = B * S, held + S
        xh, wh = torch.randn(N, WIDTH, device=dev).half(), torch.ones(WIDTH, device=dev).half()
        oh = torch.empty_like(xh)
        add("lowbit_rms_norm", phase, timer(lambda: ggml.lowbit_rms_norm(xh, wh, 1e-5, oh, st())), N * WIDTH * 4)
        qh = torch.randn(B, HEADS, S, DIM, device=dev).half()
        kh = torch.randn(B, KV_HEADS, S, DIM, device=dev).half()
        invf = torch.tensor([10000.0 ** (-2.0 * i / DIM) for i in range(DIM // 2)], device=dev)
        posid = torch.arange(held, held + S, device=dev)[None, :].expand(B, S).contiguous()
        add("lowbit_rotary", phase, timer(lambda: rotary_half_inplaced(invf, posid, qh, kh)), N * (HEADS + KV_HEADS) * DIM * 4)
        k8 = torch.randint(0, 120, (B, KV_HEADS, L, DIM), dtype=torch.uint8, device=dev)
        v8 = torch.randint(0, 120, (B, KV_HEADS, L, DIM), dtype=torch.uint8, device=dev)
        if S == 1:
            add("lowbit_sdp_fp8", phase, timer(lambda: kv.sdp_fp8(qh, k8, v8, None, DIM ** -0.5, False)), bytes_=B * KV_HEADS * L * 2 * DIM)
        else:
            add("lowbit_sdp_fp8_prefill", phase, timer(lambda: kv.sdp_fp8_prefill(qh, k8, v8, None, DIM ** -0.5, True)),
                flops=4.0 * DIM * (S * (S + 1) / 2) * HEADS * B)
    return rows


def run(args):
    import torch
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.bfloat16
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        src = "MEASURED_PEAKS.json"
    except (OSError, ValueError):
        peaks, src = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"
    timer = Timer(dev)
    out = {"arch": "zafepel", "dtype": "bf16", "data": "synthetic (random weights)", "peaks": {"hbm_gbs": peaks["hbm_gbs"],
           "bf16_tflops": peaks["bf16_tflops"], "source": src},
           "config": {"width": WIDTH, "ff": FF, "layers": LAYERS, "layer_runs": LAYERS + 2, "heads": HEADS, "kv_heads": KV_HEADS, "dim": DIM,
                      "window": WINDOW, "gla": [G_HEADS, G_DIM, G_VDIM], "vocab": VOCAB, "cache": "256 MB rewritten between timed runs"}}
    model = build_zafepel(dev, dtype)
    out["zafepel"] = [throughput(model, dev, timer, b) for b in (1, 8)]
    del model
    torch.cuda.empty_cache()
    if not args.no_compare:
        model = build_zafepel(dev, dtype, low_bit="sym_int4")
        out["zafepel_sym_int4"] = [throughput(model, dev, timer, b) for b in (1, 8)]
        del model
        torch.cuda.empty_cache()
        model = build_llama(dev, torch.float16)
        out["llama_equal_size"] = [throughput(model, dev, timer, b) for b in (1, 8)]
        out["llama_equal_size_note"] = "sym_int4 weights, FP8 KV cache, fp16 activations, same width / ff / heads / layer runs"
        del model
        torch.cuda.empty_cache()
    out["kernels"] = kernel_table(dev, dtype, peaks, timer)
    print(json.dumps(out))
