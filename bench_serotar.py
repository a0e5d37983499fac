"""`python bench.py --arch serotar`: the Serotar design at layer sizes of a real model (random weights), beside a Mixtral of equal
width, depth, head count and expert geometry served by the same framework: prefill and decode throughput through the public
API, and every kernel of the design timed alone against its roofline next to the like kernel of the Mixtral / Llama path.

Timing and rooflines as in bench_mixers.py: CUDA events on the launching stream, 3 warm-up runs, median of 7, a 256 MB buffer
rewritten between runs; algorithmic bytes / the measured copy bandwidth, or algorithmic flops / the measured bf16 GEMM burst
rate (MEASURED_PEAKS.json).  One JSON line on stdout.
"""
import json
import math
import os

from bench_mixers import NEW, PROMPT, ROOT, Timer, throughput

WIDTH, FF, VOCAB, LAYERS = 2048, 5632, 32000, 8
HEADS, DIM, VDIM, Q_RANK, KV_RANK = 16, 128, 128, 768, 512
EXPERTS, IDENTITY, TOP, GROUPS, KEEP, EXPERT_FF, SHARED_FF = 8, 2, 2, 2, 1, 2816, 2816
SIDE_DIM, BUCKETS = 64, 100003


def serotar_config():
    mixer = {"heads": HEADS, "dim": DIM, "vdim": VDIM, "q_rank": Q_RANK, "kv_rank": KV_RANK, "scale": DIM ** -0.5}
    moe = {"kind": "moe", "expert": {"ff": EXPERT_FF}, "shared": {"ff": SHARED_FF},
           "router": {"experts": EXPERTS, "identity": IDENTITY, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}}}
    layers = [{"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": FF} if i == 0 else moe} for i in range(LAYERS)]
    return {"architecture": "Serotar", "vocab": VOCAB, "width": WIDTH, "norm": {"eps": 1e-5}, "token_side": {"dim": SIDE_DIM},
            "embedding": {"scale": 1.0, "bigram": {"buckets": BUCKETS, "mul_prev": 1000003, "mul_cur": 8191}}, "layers": layers}


def build_serotar(dev, dtype):
    import torch
    from ipex_llm_b200.transformers.convert import _optimize_pre, _optimize_post
    from ipex_llm_b200.transformers.models.serotar import SerotarConfig, SerotarForCausalLM
    cfg = SerotarConfig(**serotar_config())
    with torch.device("meta"):
        model = SerotarForCausalLM(cfg)
    gen = torch.Generator(device=dev).manual_seed(0)
    for mod in model.modules():
        for name, p in list(mod._parameters.items()):
            if p is None:
                continue
            t = torch.empty(p.shape, device=dev, dtype=torch.float32)
            if p.dim() >= 2:
                t.normal_(0.0, 1.0 / math.sqrt(p.shape[-1]), generator=gen)
            elif name == "dwa":
                t.fill_(1.0 / p.shape[0])
            elif name in ("weight", "ls1", "ls2"):
                t.fill_(1.0)
            else:
                t.normal_(0.0, 0.1, generator=gen)
            mod._parameters[name] = torch.nn.Parameter(t.to(dtype), requires_grad=False)
    return _optimize_post(_optimize_pre(model.eval()))


def build_mixtral(dev, dtype):
    import torch
    import transformers
    from ipex_llm_b200.optimize import low_memory_init
    from ipex_llm.transformers import AutoModelForCausalLM
    cfg = transformers.MixtralConfig(hidden_size=WIDTH, intermediate_size=EXPERT_FF, num_hidden_layers=LAYERS, num_attention_heads=HEADS,
                                     num_key_value_heads=4, head_dim=DIM, vocab_size=VOCAB, max_position_embeddings=8192,
                                     num_local_experts=EXPERTS, num_experts_per_tok=TOP, sliding_window=None, rms_norm_eps=1e-5,
                                     tie_word_embeddings=False)
    with low_memory_init():
        model = transformers.MixtralForCausalLM(cfg)
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


def kernel_table(dev, dtype, peaks, timer, serotar, mixtral):
    """each kernel of the design alone at the layer's sizes (prefill: 1 x PROMPT tokens; decode: 8 rows, one token each, PROMPT
    cached), and the Mixtral / Llama path's like kernels at the same sizes"""
    import torch
    from ipex_llm_b200.transformers.models import mixer_ops as ops
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
    moe = serotar.model.layers[1].mlp
    for phase, B, S, held in (("prefill", 1, PROMPT, 0), ("decode", 8, 1, PROMPT)):
        N, L = B * S, held + S
        pad = torch.zeros(B, dtype=torch.int32, device=dev)
        ids = torch.randint(0, VOCAB, (B, S), device=dev)
        prev = torch.zeros(B, dtype=torch.int64, device=dev)
        core = serotar.model
        add("embed_pair", phase, timer(lambda: ops.embed_pair(core.embed_tokens.weight, 1.0, core.pair_embed.weight, BUCKETS, 1000003, 8191, ids,
                                                              prev, held, pad if held == 0 else None, dtype)),
            N * WIDTH * (2 * es + 4 + es), like="embedding gather")
        x, y, gain, ls = torch.randn(N, WIDTH, device=dev), rnd(N, WIDTH), vec(1)[0], vec(WIDTH)
        add("rms_residual", phase, timer(lambda: ops.rms_residual(x, y, gain, ls, 1e-5, dtype)), N * WIDTH * (8 + 2 * es), like="lowbit_rms_norm")
        stack, coef = torch.randn(LAYERS + 1, N, WIDTH, device=dev), vec(5)
        add("rms_residual + depth average (5 streams)", phase,
            timer(lambda: ops.rms_residual(x, y, None, ls, 1e-5, dtype, stack=stack, index=4, coef=coef)), N * WIDTH * (8 + 2 * es + 5 * 4),
            like="lowbit_rms_norm")
        proj, qw, cw = rnd(B, S, Q_RANK + KV_RANK), vec(Q_RANK), vec(KV_RANK)
        store = rnd(B, L, KV_RANK)
        add("latent_prepare", phase, timer(lambda: ops.latent_prepare(proj, 0, Q_RANK, qw, Q_RANK, KV_RANK, cw, 1e-5, store, held, 0, pad)),
            N * (Q_RANK + KV_RANK) * 2 * es, like="lowbit_rotary / rope_kv_append")
        if S > 1:
            q, kvx = rnd(N, HEADS * DIM), rnd(B, L, HEADS * (DIM + VDIM))
            k, v = kvx[..., :HEADS * DIM].view(B, L, HEADS, DIM), kvx[..., HEADS * DIM:].view(B, L, HEADS, VDIM)
            add("softmax_attention (expanded keys / values)", phase, timer(lambda: ops.softmax_attention(q, k, v, B, S, HEADS, held, 0, pad, 0, DIM ** -0.5)),
                flops=2.0 * (DIM + VDIM) * (S * (S + 1) / 2) * HEADS * B, like="lowbit_sdp_fp8_prefill")
        else:
            qa, lat = rnd(N, HEADS * KV_RANK), store.unsqueeze(2)
            add("softmax_attention (latent cache as key = value)", phase,
                timer(lambda: ops.softmax_attention(qa, lat, lat, B, S, HEADS, held, 0, pad, 0, DIM ** -0.5)), bytes_=B * L * KV_RANK * es,
                like="lowbit_sdp_fp8")
        h = rnd(N, WIDTH)
        add("grouped_router", phase, timer(lambda: ops.grouped_router(h, moe.router, moe.correction, GROUPS, KEEP, TOP)),
            N * WIDTH * es + (EXPERTS + IDENTITY) * WIDTH * es, like="router linear + softmax + topk (torch)")
        z, pq = rnd(N, FF), vec(2)
        add("xielu", phase, timer(lambda: ops.xielu(z, pq)), N * FF * 2 * es, like="silu*mul inside lowbit_mlp")
        gu = rnd(N, 2 * EXPERT_FF)
        add("silu_mul", phase, timer(lambda: ops.silu_mul(gu, EXPERT_FF)), N * EXPERT_FF * 3 * es, like="silu*mul inside lowbit_mlp")
        sg = rnd(N, SIDE_DIM)
        add("gelu_table_mul", phase, timer(lambda: ops.gelu_table_mul(sg, core.side_embed.weight, SIDE_DIM, ids.reshape(-1))), N * SIDE_DIM * 3 * es)
        idx, wgt = ops.grouped_router(h, moe.router, moe.correction, GROUPS, KEEP, TOP)
        if S == 1:
            tables = moe.address_tables(dtype, dev)
            for n in (1, 8):
                real = idx[:n][idx[:n] < EXPERTS]
                distinct, pairs = int(real.unique().numel()), int(real.numel())
                add(f"moe_small ({n} rows, {pairs} expert calls on {distinct} experts)", phase,
                    timer(lambda: ops.moe_small(h[:n], idx[:n], wgt[:n], tables[0], tables[1], EXPERT_FF, EXPERTS, EXPERTS + IDENTITY, None,
                                                ffs=tables[2])),
                    bytes_=distinct * 3 * EXPERT_FF * WIDTH * es, like="lowbit_moe (moe_forward_vec)")
        else:
            rows_ = rnd(N * TOP, WIDTH)
            pos = torch.randperm(N * TOP, device=dev).to(torch.int32)
            add("moe_combine", phase, timer(lambda: ops.moe_combine(rows_, pos, idx, wgt, h, h, EXPERTS, EXPERTS + IDENTITY)),
                N * WIDTH * (TOP * es + 2 * es + 4))
    if mixtral is None:
        return rows
    import ipex_llm_b200.ggml.model.llama.llama_cpp as ggml
    from ipex_llm_b200.transformers import kv
    st = lambda: torch.cuda.current_stream(dev).cuda_stream                                   # noqa: E731
    KVH = 4
    for phase, B, S, held in (("prefill", 1, PROMPT, 0), ("decode", 8, 1, PROMPT)):
        N, L = B * S, held + S
        xh, wh = torch.randn(N, WIDTH, device=dev).half(), torch.ones(WIDTH, device=dev).half()
        oh = torch.empty_like(xh)
        add("lowbit_rms_norm", phase, timer(lambda: ggml.lowbit_rms_norm(xh, wh, 1e-5, oh, st())), N * WIDTH * 4)
        qh = torch.randn(B, HEADS, S, DIM, device=dev).half()
        k8 = torch.randint(0, 120, (B, KVH, L, DIM), dtype=torch.uint8, device=dev)
        v8 = torch.randint(0, 120, (B, KVH, L, DIM), dtype=torch.uint8, device=dev)
        if S == 1:
            add("lowbit_sdp_fp8", phase, timer(lambda: kv.sdp_fp8(qh, k8, v8, None, DIM ** -0.5, False)), bytes_=B * KVH * L * 2 * DIM)
        else:
            add("lowbit_sdp_fp8_prefill", phase, timer(lambda: kv.sdp_fp8_prefill(qh, k8, v8, None, DIM ** -0.5, True)),
                flops=4.0 * DIM * (S * (S + 1) / 2) * HEADS * B)
    experts = mixtral.model.layers[0].mlp.experts
    x1 = torch.randn(1, WIDTH, device=dev).half()
    i1, w1 = torch.tensor([[1, 5]], device=dev), torch.tensor([[0.6, 0.4]], device=dev).half()
    add("lowbit_moe (moe_forward_vec, 1 row, 2 experts, sym_int4)", "decode", timer(lambda: experts.fused_one_token(x1, i1, w1)),
        bytes_=2 * 3 * EXPERT_FF * WIDTH * 0.5625)
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
    out = {"arch": "serotar", "dtype": "bf16", "data": "synthetic (random weights)",
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": src},
           "config": {"width": WIDTH, "dense_ff": FF, "layers": LAYERS, "heads": HEADS, "dim": DIM, "vdim": VDIM, "q_rank": Q_RANK,
                      "kv_rank": KV_RANK, "experts": EXPERTS, "identity": IDENTITY, "top": TOP, "expert_ff": EXPERT_FF, "shared_ff": SHARED_FF,
                      "vocab": VOCAB, "prompt": PROMPT, "new_tokens": NEW, "cache": "256 MB rewritten between timed runs"}}
    serotar = build_serotar(dev, dtype)
    out["serotar"] = [throughput(serotar, dev, timer, b) for b in (1, 8)]
    out["serotar_recorded_step_failed"] = serotar.__dict__.get("_b200_state_graph_failed")
    mixtral = None
    if not args.no_compare:
        mixtral = build_mixtral(dev, torch.float16)
        out["mixtral_equal_size"] = [throughput(mixtral, dev, timer, b) for b in (1, 8)]
        out["mixtral_equal_size_note"] = "sym_int4 weights, FP8 KV cache, fp16 activations, same width / layers / heads / experts / top"
    out["kernels"] = kernel_table(dev, dtype, peaks, timer, serotar, mixtral)
    print(json.dumps(out))
