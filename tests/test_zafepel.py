"""The Zafepel design in the framework against the plain statements of tests/zafepel_oracle.py (float64).

CPU tests cover what needs no kernel: the configuration's layer order, the checkpoint reader and name map, the merged
projections, the cache's bookkeeping.  GPU tests run the kernels (there is no CPU path): every mechanism alone on odd sizes,
whole prompts against token-by-token decoding and against prompts fed in portions, unequal batches against each request alone,
rows leaving a batch, storage that is trimmed and used again, keys just inside and just outside the window, far tokens that only
the recurrent state remembers, long decoding, and greedy generation through ``generate()``.
"""
import json
import math
import os

import pytest
import torch

import zafepel_oracle as O

F64 = torch.float64


# ------------------------------------------------------------------ helpers
def save_checkpoint(cfg, weights, folder):
    """config.json + model.safetensors (8-byte header length, JSON header, raw data)"""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32"}
    header, blobs, off = {}, [], 0
    for k, v in weights.items():
        raw = v.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        header[k] = {"dtype": names[v.dtype], "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(len(h).to_bytes(8, "little"))
        f.write(h)
        for b in blobs:
            f.write(b)


def load_framework(folder, dtype, device=None):
    from ipex_llm_b200.transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(str(folder), torch_dtype=dtype)
    return model.to(device) if device is not None else model


def logits_error(got, want):
    """per position: rms over the vocabulary of the difference (mean removed) over the rms of the wanted logits"""
    d = got.to(F64) - want.to(F64)
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / want.to(F64).pow(2).mean().sqrt()).max().item()


def oracle_logits(cfg, w, tokens):
    om = O.OracleModel(cfg, w)
    return om.forward(torch.tensor([tokens]), om.new_state())[0]


@pytest.fixture(scope="module")
def mixers(cuda_device):
    from ipex_llm_b200.transformers.models import mixer_ops
    return mixer_ops


CONFIGS = {
    # sizes chosen so that nothing coincides: dim != vdim, rotary narrower than the head, grouped heads on both sides,
    # a repeated block that does not start at layer 0, layers with and without a feed-forward
    "odd": dict(),
    # one head per group, full-width rotary, two taps, a block repeated three times from layer 0, no cap on the logits
    "plain": dict(width=48, vocab=61, order=("gla", "parallel"), loop=(0, 2, 3), window=3, heads=2, kv_heads=2, dim=8, vdim=8,
                  rot_dims=8, r_heads=2, r_kv_heads=2, r_dim=8, r_vdim=8, taps=2, g_heads=1, g_dim=8, g_vdim=8, rank=3, ff=24,
                  mlp_on=(False, True), softcap=None),
    # no repeated block at all, a convolution of one tap, a window longer than the test's sequences, wide heads
    "flat": dict(width=64, vocab=50, order=("parallel", "parallel", "gla"), loop=None, window=64, heads=6, kv_heads=1, dim=20,
                 vdim=36, rot_dims=6, r_heads=6, r_kv_heads=3, r_dim=40, r_vdim=12, taps=1, g_heads=2, g_dim=33, g_vdim=70, rank=9,
                 ff=72, mlp_on=(True, True, False)),
    # head sizes that tile into 16s (the tensor-core attention of a 16-bit model), a window shorter than a 64-row block,
    # two passes of a three-layer block that ends at the last layer
    "tile": dict(width=96, vocab=83, order=("gla", "parallel", "parallel"), loop=(0, 3, 2), window=21, heads=4, kv_heads=1, dim=32,
                 vdim=48, rot_dims=32, r_heads=2, r_kv_heads=1, r_dim=32, r_vdim=16, taps=3, g_heads=2, g_dim=16, g_vdim=32, rank=6,
                 ff=64, mlp_on=(True, False, False)),
}


def make(name, seed=0):
    cfg = O.random_config(seed, **CONFIGS[name])
    w = O.random_weights(cfg, seed + 1)
    return cfg, w


# ================================================================== CPU: configuration, loader, cache bookkeeping
def test_layer_runs_follow_the_loop():
    from ipex_llm_b200.transformers.models.zafepel import ZafepelConfig
    layers = [{"type": "gla", "mixer": {}, "mlp": None}] * 5
    c = ZafepelConfig(layers=layers, loop={"start": 1, "stop": 3, "times": 3})
    assert c.layer_runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None), (4, None)]
    assert ZafepelConfig(layers=layers, loop=None).layer_runs() == [(i, None) for i in range(5)]
    assert ZafepelConfig(layers=layers, loop={"start": 0, "stop": 5, "times": 1}).layer_runs()[0] == (0, 0)
    cfg, w = make("odd")
    assert [r for r, _ in ZafepelConfig(**cfg).layer_runs()] == O.OracleModel(cfg, w).runs


def test_loader_maps_every_tensor_and_merges(tmp_path):
    from ipex_llm_b200.transformers.models.zafepel import read_safetensors
    cfg, w = make("odd")
    save_checkpoint(cfg, w, tmp_path)
    back = read_safetensors(os.path.join(tmp_path, "model.safetensors"))
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    model = load_framework(tmp_path, torch.bfloat16)
    assert type(model).__name__ == "ZafepelForCausalLM" and model.config.model_type == "zafepel"
    mx = model.model.layers[0].mixer
    l, r = cfg["layers"][0]["mixer"]["left"], cfg["layers"][0]["mixer"]["right"]
    rows = (l["heads"] + l["kv_heads"]) * l["dim"] + l["kv_heads"] * l["vdim"] + 2 * r["kv_heads"] * r["dim"] \
        + 2 * r["heads"] * r["vdim"] + 2 * r["heads"]
    assert mx.in_proj.weight.shape == (rows, cfg["width"]) and not hasattr(mx.left, "q_proj")
    nq = l["heads"] * l["dim"]
    assert torch.equal(mx.in_proj.weight[:nq], w["l0.mix.left.q"]) and torch.equal(mx.in_proj.bias[:nq], w["l0.mix.left.q.b"])
    assert float(mx.in_proj.bias[-1]) == 0.0                       # the delta-rule projections have no bias
    assert torch.equal(mx.out_proj.weight[:, :l["heads"] * l["vdim"]], w["l0.mix.left.o"])
    assert torch.equal(mx.out_proj.weight[:, l["heads"] * l["vdim"]:], w["l0.mix.right.o"])
    g = model.model.layers[1].mixer
    assert g.in_proj.weight.shape[0] == 2 * 3 * 7 + 2 * 3 * 5 + w["l1.mix.a1"].shape[0] and not hasattr(g, "a1_proj")
    assert torch.equal(model.model.loop_step, w["loop.step"])
    # a tensor of the wrong shape is refused, by name
    bad = dict(w)
    bad["l0.mix.left.pb"] = torch.zeros(3, dtype=torch.bfloat16)
    save_checkpoint(cfg, bad, tmp_path / "bad")
    with pytest.raises(RuntimeError, match="pos_bias"):
        load_framework(tmp_path / "bad", torch.bfloat16)


def test_state_cache_bookkeeping():
    from ipex_llm_b200.transformers import kv
    cache = kv.DynamicStateCache()
    mask = torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 1], [0, 0, 0, 0, 1]])
    cache.start(mask, 3, 5, torch.device("cpu"))
    assert cache.pad.tolist() == [2, 0, 4]
    with pytest.raises(RuntimeError, match="left padding"):
        kv.DynamicStateCache().start(torch.tensor([[1, 0, 1]]), 1, 3, torch.device("cpu"))
    st = cache.run_state(2, window=4)
    like = torch.empty(3, 2, 0, 6)
    k, v, held = st.kv.slots(like, like, 5)
    assert held == 0 and st.kv.capacity() >= 5
    assert k.shape == (3, 2, st.kv.capacity(), 6) and k.is_contiguous()
    k[:, :, :5] = torch.arange(5.0)[None, None, :, None]
    st.kv.commit(5)
    cache.advance(5)
    assert cache.get_seq_length() == 5 and st.kv.keys.shape[2] == 5
    st.rec.matrix(3, 2, 4, 4, torch.device("cpu"))[:] = torch.arange(3.0)[:, None, None, None]
    cache.batch_select_indices([2, 0])
    assert cache.pad.tolist() == [4, 2] and st.rec.state[:, 0, 0, 0].tolist() == [2.0, 0.0]
    assert st.kv.keys.shape == (2, 2, 5, 6) and st.kv.keys[0, 0, :, 0].tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]
    # trimming keeps the last window - 1 positions and remembers how many slots left the storage
    old_block, kv.KV_ALLOC_BLOCK_LENGTH = kv.KV_ALLOC_BLOCK_LENGTH, 2
    try:
        k, v, held = st.kv.slots(like[:2], like[:2], 20)
        k[:, :, 5:25] = torch.arange(5.0, 25.0)[None, None, :, None]
        st.kv.commit(20)
        cache.advance(20)
        assert st.kv.dropped == 22 and st.kv.keys[1, 1, :, 3].tolist() == [22.0, 23.0, 24.0]
        assert cache.seen - st.kv.keys.shape[2] == st.kv.dropped
    finally:
        kv.KV_ALLOC_BLOCK_LENGTH = old_block


def test_registry_picks_the_design(tmp_path):
    from ipex_llm_b200.transformers.model import native_architecture
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Zafepel"}))
    assert native_architecture(tmp_path).endswith("models.zafepel")
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama", "architectures": ["LlamaForCausalLM"]}))
    assert native_architecture(tmp_path) is None


# ================================================================== GPU: each mechanism alone
def _rand(shape, gen, dtype, device, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype).to(device)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dyt_polynorm_softcap_gated_norm(mixers, cuda_device, dtype):
    from ipex_llm_b200.transformers.models.zafepel import DynamicTanh
    g = torch.Generator().manual_seed(3)
    n, w = 7, 45
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    x = torch.randn(n, w, generator=g)
    y = _rand((n, w), g, dtype, cuda_device, 2.0)
    add = _rand((w,), g, dtype, cuda_device)
    post, pre = DynamicTanh(w), DynamicTanh(w)
    for m in (post, pre):
        for p in m.parameters():
            p.data = torch.randn(p.shape, generator=g) * 0.5 + 0.8
        m.to(dtype).to(cuda_device)
    xd = x.clone().to(cuda_device)
    h = mixers.dyt_residual_norm(xd, (y, post), add, pre, dtype)
    want_x = x.to(F64) + O.dyn_tanh(y.cpu().to(F64), post.alpha.cpu().to(F64), post.weight.cpu().to(F64), post.bias.cpu().to(F64)) + add.cpu().to(F64)
    want_h = O.dyn_tanh(want_x, pre.alpha.cpu().to(F64), pre.weight.cpu().to(F64), pre.bias.cpu().to(F64))
    assert (xd.cpu().to(F64) - want_x).abs().max() < 1e-5            # the residual is 32-bit whatever the dtype
    assert (h.cpu().to(F64) - want_h).abs().max() < tol * 3
    x2 = x.clone().to(cuda_device)
    assert mixers.dyt_residual_norm(x2, (y, post), None, None, dtype) is None and not torch.equal(x2.cpu(), x)
    # PolyNorm
    z = _rand((n, 53), g, dtype, cuda_device, 1.5)
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1]).to(dtype).to(cuda_device)
    got = mixers.poly_norm(z, coef, 1e-5).cpu().to(F64)
    want = O.poly_norm(z.cpu().to(F64), coef.cpu().to(F64), 1e-5)
    assert (got - want).abs().max() < tol * want.abs().max()
    # soft cap (and its absence)
    lg = _rand((n, 31), g, dtype, cuda_device, 20.0)
    assert (mixers.soft_cap(lg, 15.0).cpu().to(F64) - O.soft_cap(lg.cpu().to(F64), 15.0)).abs().max() < 1e-4
    assert torch.equal(mixers.soft_cap(lg, None).cpu(), lg.cpu().float())
    # gated RMS norm into a column range of a wider buffer, scaled
    H, Dv, ld = 3, 13, 70
    o = torch.randn(n, H, Dv, generator=g)
    gate = _rand((n, ld), g, dtype, cuda_device)
    wv = _rand((Dv,), g, dtype, cuda_device)
    out = torch.zeros(n, 50, dtype=dtype, device=cuda_device)
    mixers.gated_rms_norm(o.to(cuda_device), gate, 9, wv, 1e-5, out, 4, 0.6)
    want = 0.6 * O.rms_unit(o.to(F64), 1e-5) * wv.cpu().to(F64) * O.silu(gate.cpu().to(F64)[:, 9:9 + H * Dv].view(n, H, Dv))
    assert (out.cpu().to(F64)[:, 4:4 + H * Dv] - want.reshape(n, -1)).abs().max() < tol * 3
    assert float(out[:, :4].abs().max()) == 0.0 and float(out[:, 4 + H * Dv:].abs().max()) == 0.0


def _attention_case(mixers, device, dtype, B, S, held, pad, H, G, D, Dv, rot_dims, window, seed, shift=0, q_gain=None):
    """runs prepare + attention on new tokens behind ``held`` cached ones; returns (got, want) [B, S, H * Dv]"""
    g = torch.Generator().manual_seed(seed)
    cap = held + S + 3
    P = 5 + H * D + G * D + G * Dv
    total = held + S
    proj_all = torch.randn(B, total, P, generator=g).to(dtype)
    if q_gain is not None:
        q_gain(proj_all)
    qw, kw = (torch.rand(D, generator=g) + 0.5).to(dtype), (torch.rand(D, generator=g) + 0.5).to(dtype)
    hb = (torch.randn(H, generator=g) - 0.5).to(dtype)
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)] or [0.0], dtype=F64)
    pad_t = torch.tensor(pad, dtype=torch.int32)
    oq, ok, ov = 5, 5 + H * D, 5 + H * D + G * D
    scale = 1.3 / math.sqrt(D)
    # oracle on every slot at once
    p = proj_all.to(F64)
    q = O.rms_unit(p[..., oq:ok].view(B, total, H, D), 1e-5) * qw.to(F64)
    k = O.rms_unit(p[..., ok:ov].view(B, total, G, D), 1e-5) * kw.to(F64)
    v = p[..., ov:].view(B, total, G, Dv)
    pos = (shift + torch.arange(total))[None, :] - pad_t[:, None].long()
    q = O.rotate_pairs(q, pos, 50.0, rot_dims)
    k = O.rotate_pairs(k, pos, 50.0, rot_dims)
    want = O.sigmoid_window_attention(q[:, held:], k, v, held, pad_t.long() - shift, window, scale, hb.to(F64)).reshape(B, S, H * Dv)
    # the kernels: first the cached part, then the new tokens
    ks = torch.zeros(B, G, cap, D, dtype=dtype, device=device)
    vs = torch.zeros(B, G, cap, Dv, dtype=dtype, device=device)
    dev = lambda t: t.to(device)
    out = torch.empty(B * S, H * Dv + 2, dtype=dtype, device=device)
    for lo, n in ((0, held), (held, S)):
        if n == 0:
            continue
        qq = mixers.window_qk_prepare(dev(proj_all[:, lo:lo + n].contiguous()), oq, ok, ov, H, G, D, Dv, dev(qw), dev(kw), 1e-5,
                                      dev(inv_freq), rot_dims, ks, vs, cap, lo, shift, dev(pad_t))
    mixers.sigmoid_window_attention(qq, ks, vs, cap, held, shift, dev(pad_t), window, scale, dev(hb), out, 1, 1.0)
    return out[:, 1:1 + H * Dv].view(B, S, H * Dv).cpu().to(F64), want


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("S,held", [(11, 0), (1, 9), (4, 6), (1, 0)])
def test_window_attention_alone(mixers, cuda_device, dtype, tol, S, held):
    got, want = _attention_case(mixers, cuda_device, dtype, B=2, S=S, held=held, pad=[0, 3 if held + S > 3 else 0], H=6, G=2, D=10, Dv=7,
                                rot_dims=6, window=4, seed=5)
    assert (got - want).abs().max() < tol * max(1.0, want.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("D,Dv,window,S,held", [(7, 300, 1, 20, 0), (300, 5, 2, 3, 40), (36, 520, 50, 33, 10), (2, 1, 3, 9, 0)])
def test_window_attention_extreme_sizes_fp32(mixers, cuda_device, D, Dv, window, S, held):
    """a window of one token (only itself), more value columns than one pass holds, heads wider than a warp's turn"""
    got, want = _attention_case(mixers, cuda_device, torch.float32, B=2, S=S, held=held, pad=[1, 0], H=2, G=1, D=D, Dv=Dv,
                                rot_dims=2 if D >= 2 else 0, window=window, seed=D)
    assert (got - want).abs().max() < 3e-5 * max(1.0, want.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,Dv,H,G", [(48, 32, 4, 2), (128, 128, 2, 1), (32, 80, 3, 3), (160, 16, 2, 2), (256, 256, 1, 1), (24, 264, 2, 1)])
@pytest.mark.parametrize("S,held,window", [(70, 50, 40), (130, 0, 300), (16, 3, 7), (1, 300, 290), (5, 40, 33), (1, 6, 9)])
def test_window_attention_many_tokens_16bit(mixers, cuda_device, dtype, D, Dv, H, G, S, held, window):
    """the tensor-core path (16 tokens or more): head sizes that tile into 16s, portions that end inside a 64-row block, windows
    shorter and longer than a block, padding, a filled cache in front; and the general kernel's 16-byte loads on the same head
    sizes when a few tokens are decoded"""
    got, want = _attention_case(mixers, cuda_device, dtype, B=2, S=S, held=held, pad=[0, 5], H=H, G=G, D=D, Dv=Dv, rot_dims=16,
                                window=window, seed=D + S)
    # keys and queries are rounded to 16 bits on the way (2^-9 relative each); the weights keep 16 bits
    assert (got - want).abs().max() < 2e-2 * max(1.0, want.abs().max())
    assert (got - want).pow(2).mean().sqrt() < 4e-3 * want.pow(2).mean().sqrt().clamp(min=0.1)


@pytest.mark.gpu
@pytest.mark.parametrize("held,S", [(0, 40), (39, 1)])            # the edge inside a prompt, and met by a decoded token
def test_window_edge_decides(mixers, cuda_device, held, S):
    """every key but one scores far below zero (weight ~ 0); the one that stands out sits either at distance window - 1
    (seen: the output is its value) or at distance window (not seen: the output is ~ 0)"""
    H = G = 1
    D, Dv, window, total = 8, 4, 7, 40

    def run(distance):
        def gain(proj):
            proj[..., 5:5 + 2 * D] = 0.0
            proj[..., 5 + D - 1] = 1.0                             # every query: e_last  (norm keeps the direction)
            proj[..., 5 + D + D - 1] = -1.0                        # every key: -e_last -> score very negative
            proj[:, total - 1 - distance, 5 + D + D - 1] = 1.0     # the chosen key
        return _attention_case(mixers, cuda_device, torch.float32, B=1, S=S, held=held, pad=[0], H=H, G=G, D=D, Dv=Dv, rot_dims=0,
                               window=window, seed=11, q_gain=gain)

    # scale * |q||k| = 1.3 / sqrt(8) * 8 = 3.7, bias ~ -0.5: sigmoid(3.2) = 0.96 against sigmoid(-4.2) = 0.015 per other key
    inside, want_in = run(window - 1)
    outside, want_out = run(window)
    assert (inside - want_in).abs().max() < 1e-4 and (outside - want_out).abs().max() < 1e-4
    assert (want_in[0, -1] - want_out[0, -1]).abs().max() > 0.3   # the two cases really differ at the last token


@pytest.mark.gpu
def test_window_attention_after_trim(mixers, cuda_device):
    """storage whose first slots were dropped (shift > 0) and rows whose padding lies before the storage"""
    got, want = _attention_case(mixers, cuda_device, torch.float32, B=2, S=3, held=6, pad=[0, 102], H=2, G=1, D=6, Dv=5, rot_dims=4,
                                window=5, seed=8, shift=100)
    assert (got - want).abs().max() < 2e-5 * max(1.0, want.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("taps", [1, 2, 4, 9])
def test_short_conv_in_portions(mixers, cuda_device, dtype, tol, taps):
    g = torch.Generator().manual_seed(taps)
    B, total, C, off, P = 2, 13, 11, 3, 20
    proj = torch.randn(B, total, P, generator=g).to(dtype)
    w = torch.randn(C, taps, generator=g).to(dtype)
    pad = torch.tensor([0, 2], dtype=torch.int32)
    want, _ = O.short_conv_silu(proj.to(F64)[..., off:off + C], w.to(F64), torch.zeros(B, taps - 1, C, dtype=F64), 0, pad.long())
    tail = torch.zeros(B, max(taps - 1, 1), C, dtype=dtype, device=cuda_device)
    nxt = torch.empty_like(tail)
    got, at = [], 0
    for n in (1, 2, 5, 1, 4):                                      # portions shorter and longer than the taps
        y = mixers.short_conv_silu(proj[:, at:at + n].contiguous().to(cuda_device), off, C, w.to(cuda_device), tail, nxt, at, pad.to(cuda_device))
        tail, nxt = nxt, tail
        got.append(y.cpu())
        at += n
    got = torch.cat(got, 1).to(F64)
    for b in range(B):
        lo = int(pad[b])
        assert (got[b, lo:] - want[b, lo:]).abs().max() < tol * max(1.0, want.abs().max())


def _delta_inputs(B, total, G, H, D, Dv, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    conv = torch.randn(B, total, 2 * G * D + H * Dv, generator=g).to(dtype)
    proj = torch.randn(B, total, 2 * H + 3, generator=g).to(dtype)
    A_log, dtb = (torch.randn(H, generator=g) * 0.5 - 1).to(dtype), (torch.randn(H, generator=g) * 0.5).to(dtype)
    return conv, proj, A_log, dtb


def _delta_oracle(conv, proj, A_log, dtb, G, H, D, Dv, pad):
    B, total, _ = conv.shape
    c, p = conv.to(F64), proj.to(F64)
    q = O.unit_vector(c[..., :G * D].view(B, total, G, D)) * D ** -0.5
    k = O.unit_vector(c[..., G * D:2 * G * D].view(B, total, G, D))
    v = c[..., 2 * G * D:].view(B, total, H, Dv)
    beta = torch.sigmoid(p[..., 1:1 + H])
    decay = torch.exp(-torch.exp(A_log.to(F64)) * torch.nn.functional.softplus(p[..., 1 + H:1 + 2 * H] + dtb.to(F64)))
    return O.gated_delta_rule(q, k, v, beta, decay, torch.zeros(B, H, D, Dv, dtype=F64), 0, pad.long())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-5)])     # inputs are rounded, the recurrence is 32-bit
@pytest.mark.parametrize("G,H,D,Dv", [(1, 3, 5, 9), (2, 2, 40, 33), (2, 4, 16, 130), (1, 1, 70, 3), (1, 2, 200, 20), (1, 1, 600, 40),
                                       (1, 1, 1024, 8)])
def test_delta_rule_alone_and_in_portions(mixers, cuda_device, dtype, tol, G, H, D, Dv):
    B, total = 2, 37
    conv, proj, A_log, dtb = _delta_inputs(B, total, G, H, D, Dv, 17, dtype)
    pad = torch.tensor([0, 5], dtype=torch.int32)
    want_o, want_s = _delta_oracle(conv, proj, A_log, dtb, G, H, D, Dv, pad)
    dev = lambda t: t.to(cuda_device)
    for portions in ((total,), (1, 2, 17, 1, 16), tuple([1] * total)):
        state = torch.zeros(B, H, D, Dv, device=cuda_device)
        got, at = [], 0
        for n in portions:
            got.append(mixers.gated_delta_rule(dev(conv[:, at:at + n].contiguous()), G, H, D, Dv, dev(proj[:, at:at + n].contiguous()), 1, 1 + H,
                                               dev(A_log), dev(dtb), state, at, dev(pad)).cpu())
            at += n
        got = torch.cat(got, 1).to(F64)
        scale = max(1.0, want_o.abs().max())
        assert (got - want_o).abs().max() < tol * 10 * scale
        assert (state.cpu().to(F64) - want_s).abs().max() < tol * 10 * max(1.0, want_s.abs().max())


@pytest.mark.gpu
def test_delta_rule_remembers_a_far_token(mixers, cuda_device):
    """token 0 writes value v0 under key e0; 500 tokens follow whose keys are orthogonal to e0 and whose decay is ~1; the last
    token asks with e0 and must read v0 back (a state that was lost or reset on the way reads ~0)"""
    G = H = 1
    D, Dv, total = 6, 5, 502
    conv = torch.zeros(1, total, 2 * D + Dv)
    conv[0, :, D + 1] = 1.0                                        # keys e1 ...
    conv[0, :, 1] = 1.0                                            # ... and queries e1 in between
    conv[0, 0, D + 1], conv[0, 0, D] = 0.0, 1.0                    # token 0: key e0
    v0 = torch.tensor([0.5, -1.0, 2.0, 0.25, -0.75])
    conv[0, 0, 2 * D:] = v0
    conv[0, -1, 1], conv[0, -1, 0] = 0.0, 1.0                      # the last token asks with e0
    proj = torch.zeros(1, total, 5)
    proj[..., 1] = 20.0                                            # beta ~ 1
    proj[..., 2] = -30.0                                           # softplus(-30) ~ 1e-13: decay ~ 1
    A_log, dtb = torch.zeros(1), torch.zeros(1)
    state = torch.zeros(1, H, D, Dv, device=cuda_device)
    dev = lambda t: t.to(cuda_device)
    o1 = mixers.gated_delta_rule(dev(conv[:, :300].contiguous()), G, H, D, Dv, dev(proj[:, :300].contiguous()), 1, 2, dev(A_log), dev(dtb),
                                 state, 0, dev(torch.zeros(1, dtype=torch.int32)))
    o2 = mixers.gated_delta_rule(dev(conv[:, 300:].contiguous()), G, H, D, Dv, dev(proj[:, 300:].contiguous()), 1, 2, dev(A_log), dev(dtb),
                                 state, 300, dev(torch.zeros(1, dtype=torch.int32)))
    assert (o2[0, -1, 0].cpu() * D ** 0.5 - v0).abs().max() < 1e-3
    assert o1[0, 5, 0].cpu().abs().max() < 1e-6                    # in between, e1 reads nothing of token 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv", [(3, 7, 5), (1, 33, 70), (2, 64, 16), (1, 300, 24), (1, 520, 136)])
def test_gated_linear_attention_alone_and_in_portions(mixers, cuda_device, dtype, H, D, Dv):
    g = torch.Generator().manual_seed(23)
    B, total, tau = 2, 29, 6.0
    P = 2 * H * D + H * Dv + 4
    proj = torch.randn(B, total, P, generator=g).to(dtype)
    z = (torch.randn(B, total, H * D, generator=g) * 3).to(dtype)
    pad = torch.tensor([4, 0], dtype=torch.int32)
    p = proj.to(F64)
    q = (p[..., :H * D] * D ** -0.5).view(B, total, H, D)
    k = p[..., H * D:2 * H * D].view(B, total, H, D)
    v = p[..., 2 * H * D:2 * H * D + H * Dv].view(B, total, H, Dv)
    alpha = (torch.sigmoid(z.to(F64)) ** (1 / tau)).view(B, total, H, D)
    want_o, want_s = O.gated_linear_attention(q, k, v, alpha, torch.zeros(B, H, D, Dv, dtype=F64), 0, pad.long())
    dev = lambda t: t.to(cuda_device)
    for portions in ((total,), (2, 1, 20, 6), tuple([1] * total)):
        state = torch.zeros(B, H, D, Dv, device=cuda_device)
        got, at = [], 0
        for n in portions:
            got.append(mixers.gated_linear_attention(dev(proj[:, at:at + n].contiguous()), H, D, Dv, dev(z[:, at:at + n].contiguous()), tau,
                                                     state, at, dev(pad)).cpu())
            at += n
        got = torch.cat(got, 1).to(F64)
        assert (got - want_o).abs().max() < 1e-4 * max(1.0, want_o.abs().max())
        assert (state.cpu().to(F64) - want_s).abs().max() < 1e-4 * max(1.0, want_s.abs().max())


# ================================================================== GPU: whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory, cuda_device):
    built = {}

    def get(name, dtype):
        key = (name, dtype)
        if key not in built:
            cfg, w = make(name)
            folder = tmp_path_factory.mktemp(f"zafepel_{name}")
            save_checkpoint(cfg, w, folder)
            built[key] = (cfg, w, load_framework(folder, dtype, cuda_device))
        return built[key]

    return get


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "plain", "flat", "tile"])
def test_whole_prompt_matches_the_oracle_fp32(models, cuda_device, name):
    cfg, w, model = models(name, torch.float32)
    toks = _tokens(cfg, 23, 1)
    want = oracle_logits(cfg, w, toks)
    model.collect_residual = []
    with torch.no_grad():
        got = model(input_ids=torch.tensor([toks], device=cuda_device)).logits[0].cpu()
    residual, model.collect_residual = model.collect_residual, None
    assert logits_error(got, want) < 2e-5
    # the residual stream after every layer run, too (a looped layer counts each time)
    om = O.OracleModel(cfg, w)
    runs = []
    om.forward(torch.tensor([toks]), om.new_state(), collect=runs)
    assert len(residual) == len(runs)
    for a, b in zip(residual, runs):
        assert (a[0].cpu().to(F64) - b[0]).abs().max() < 1e-4 * b.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "plain", "tile"])
def test_whole_prompt_matches_the_oracle_bf16(models, cuda_device, name):
    cfg, w, model = models(name, torch.bfloat16)
    toks = _tokens(cfg, 90 if name == "tile" else 23, 1)
    want = oracle_logits(cfg, w, toks)
    with torch.no_grad():
        got = model(input_ids=torch.tensor([toks], device=cuda_device)).logits[0].cpu()
    assert logits_error(got, want) < 0.06
    # and fed as a long portion, a few tokens, then one by one: the same within 16-bit rounding
    if name == "tile":
        again = _run_in_portions(model, toks, [70, 5] + [1] * 15, cuda_device)
        assert logits_error(again, want) < 0.06


def _run_in_portions(model, toks, portions, device):
    out, cache, at = [], None, 0
    with torch.no_grad():
        for n in portions:
            r = model(input_ids=torch.tensor([toks[at:at + n]], device=device), past_key_values=cache)
            cache = r.past_key_values
            out.append(r.logits[0].cpu())
            at += n
    return torch.cat(out, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "plain", "flat"])
def test_decoding_and_portions_match_the_whole_prompt(models, cuda_device, name):
    """token-by-token through the cache, portions down to two tokens, and a window that passes over decoded tokens"""
    cfg, w, model = models(name, torch.float32)
    toks = _tokens(cfg, 31, 2)
    want = oracle_logits(cfg, w, toks)
    for portions in ([31], [1] * 31, [20] + [1] * 11, [2, 3, 2, 7, 1, 16], [1, 30]):
        got = _run_in_portions(model, toks, portions, cuda_device)
        assert logits_error(got, want) < 2e-5, portions


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 0.06)])
def test_unequal_batch_matches_each_request_alone(models, cuda_device, dtype, tol):
    """left-padded rows of very different lengths (one of a single token), decoded together; a row leaves the batch on the way"""
    cfg, w, model = models("odd", dtype)
    lengths, new = [1, 9, 4, 17], 6
    rows = [_tokens(cfg, n + new, 10 + i) for i, n in enumerate(lengths)]
    want = [oracle_logits(cfg, w, r) for r in rows]
    width = max(lengths)
    ids = torch.zeros(len(rows), width, dtype=torch.int64)
    mask = torch.zeros(len(rows), width, dtype=torch.int64)
    for i, n in enumerate(lengths):
        ids[i, width - n:] = torch.tensor(rows[i][:n])
        mask[i, width - n:] = 1
    with torch.no_grad():
        r = model(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device))
        for i, n in enumerate(lengths):
            assert logits_error(r.logits[i, width - n:].cpu(), want[i][:n]) < tol, i
        cache, alive = r.past_key_values, list(range(len(rows)))
        for step in range(new):
            if step == 3:                                          # the second request ends here
                cache.batch_select_indices([0, 2, 3])
                alive = [0, 2, 3]
            nxt = torch.tensor([[rows[i][lengths[i] + step]] for i in alive], device=cuda_device)
            r = model(input_ids=nxt, past_key_values=cache)
            for j, i in enumerate(alive):
                assert logits_error(r.logits[j, 0:1].cpu(), want[i][lengths[i] + step:lengths[i] + step + 1]) < tol, (step, i)


@pytest.mark.gpu
def test_long_decoding_through_trimmed_storage(models, cuda_device, monkeypatch):
    """decoding far beyond the window with a storage that is trimmed and refilled several times on the way"""
    from ipex_llm_b200.transformers import kv
    monkeypatch.setattr(kv, "KV_ALLOC_BLOCK_LENGTH", 4)
    monkeypatch.setattr(kv.WindowKVLayer, "TRIM_FACTOR", 1)
    cfg, w, model = models("odd", torch.float32)
    toks = _tokens(cfg, 90, 3)
    want = oracle_logits(cfg, w, toks)
    got = _run_in_portions(model, toks, [12] + [1] * 50 + [7] + [1] * 21, cuda_device)
    assert logits_error(got, want) < 2e-5
    # a second batch afterwards starts from nothing (no state of the first survives in the model)
    again = _run_in_portions(model, toks[:15], [15], cuda_device)
    assert logits_error(again, want[:15]) < 2e-5


@pytest.mark.gpu
def test_greedy_generate_matches_the_oracle(models, cuda_device):
    cfg, w, model = models("odd", torch.float32)
    prompts, new = [_tokens(cfg, 5, 40), _tokens(cfg, 11, 41)], 8
    width = max(len(p) for p in prompts)
    ids = torch.zeros(2, width, dtype=torch.int64)
    mask = torch.zeros(2, width, dtype=torch.int64)
    for i, p in enumerate(prompts):
        ids[i, width - len(p):] = torch.tensor(p)
        mask[i, width - len(p):] = 1
    out = model.generate(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), max_new_tokens=new, do_sample=False, pad_token_id=0)
    # the recorded step (behind generate) and transformers' own loop on the same forward pick the same tokens
    slow = model._hf_generate(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), max_new_tokens=new, do_sample=False,
                              pad_token_id=0)
    assert torch.equal(out, slow)
    again = model.generate(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), max_new_tokens=new, do_sample=False, pad_token_id=0)
    assert torch.equal(out, again)                                 # the step's own cache starts clean every time
    om = O.OracleModel(cfg, w)
    for i, p in enumerate(prompts):
        st = om.new_state()
        lg = om.forward(torch.tensor([p]), st)
        picked, margins = [], []
        for _ in range(new):
            top = lg[0, -1].topk(2)
            picked.append(int(top.indices[0]))
            margins.append(float(top.values[0] - top.values[1]))
            lg = om.forward(torch.tensor([[picked[-1]]]), st)
        n_sure = next((j for j, m in enumerate(margins) if m < 1e-3), new)      # a tie in the oracle decides nothing
        assert out[i, width:width + n_sure].tolist() == picked[:n_sure]


@pytest.mark.gpu
def test_low_bit_conversion_save_and_load(tmp_path, cuda_device, native_lib):
    """the projections are ordinary linears to the converter: sym_int4 through from_pretrained, then save_low_bit / load_low_bit"""
    from ipex_llm_b200.transformers import AutoModelForCausalLM
    from ipex_llm_b200.transformers.low_bit_linear import LowBitLinear
    cfg = O.random_config(0, width=128, ff=192, heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, r_heads=4, r_kv_heads=2, r_dim=16,
                          r_vdim=16, g_heads=2, g_dim=16, g_vdim=32, rank=4)
    w = O.random_weights(cfg, 5)
    save_checkpoint(cfg, w, tmp_path / "m")
    toks = torch.tensor([_tokens(cfg, 19, 7)], device=cuda_device)
    dense = load_framework(tmp_path / "m", torch.bfloat16, cuda_device)
    low = AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), load_in_low_bit="sym_int4", torch_dtype=torch.bfloat16).to(cuda_device)
    converted = [n for n, m in low.named_modules() if isinstance(m, LowBitLinear)]
    assert any(n.endswith("in_proj") for n in converted) and any(n.endswith("down_proj") for n in converted) and "lm_head" in converted
    with torch.no_grad():
        a, b = dense(input_ids=toks).logits[0].cpu(), low(input_ids=toks).logits[0].cpu()
    assert torch.isfinite(b).all() and logits_error(b, a) < 0.5           # 4-bit weights: close, not equal
    low.save_low_bit(str(tmp_path / "lb"))
    back = AutoModelForCausalLM.load_low_bit(str(tmp_path / "lb")).to(cuda_device)
    with torch.no_grad():
        c = back(input_ids=toks).logits[0].cpu()
    assert logits_error(c, b) < 1e-3
