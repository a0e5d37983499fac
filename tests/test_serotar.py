"""The Serotar design in the framework against the plain statements of tests/serotar_oracle.py (float64).

CPU tests cover what needs no kernel: the configuration reader, the checkpoint's name map and the merged projections, the
registry, the latent cache's bookkeeping, the oracle's router against a brute-force statement.  GPU tests run the kernels (there
is no CPU path): every mechanism alone on odd sizes, attention through the general and the tensor-core kernel (strided keys,
grouped heads, windows decided by one outstanding key, a far key among hundreds, a future key that must stay unseen), the router
with negative choice scores, whole prompts against token-by-token decoding and against portions down to two tokens, unequal
batches against each request alone, rows leaving a batch, storage that grows past its first block, long decoding, greedy
generation through ``generate()`` (recorded step and transformers' loop) and the step's cache used again by other requests.
"""
import json
import os

import pytest
import torch

import serotar_oracle as O

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


def load_framework(folder, dtype, device=None, **kw):
    from ipex_llm_b200.transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(str(folder), torch_dtype=dtype, **kw)
    return model.to(device) if device is not None else model


def position_errors(got, want):
    """per position: rms over the vocabulary of the difference (mean removed) over the rms of the wanted logits"""
    d = got.to(F64).cpu() - want.to(F64)
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.to(F64).pow(2).mean().sqrt()


def assert_close(got, want, dtype):
    """a 32-bit model must agree everywhere; a 16-bit one may flip a routing choice that is a close call in a few places"""
    e = position_errors(got, want).reshape(-1)
    if dtype == torch.float32:
        assert e.max() < 3e-5, e.max()
    else:
        assert e.median() < 0.02 and e.quantile(0.9) < 0.15 and e.max() < 0.6, (e.median(), e.quantile(0.9), e.max())


CONFIGS = {
    # nothing coincides: dim != vdim, q_rank != kv_rank, ranks that are no multiples of 8, three kinds of layer, groups of which two
    # are kept, identity experts, every optional part present
    "odd": dict(q_rank=20, kv_rank=22),
    # everything optional absent or 1: no pair table, no side input, no layer scale, no depth average, no groups, no identity
    # experts, no shared expert, one expert per token, one head, equal head sizes
    "plain": dict(width=32, vocab=40, heads=1, dim=16, vdim=16, q_rank=8, kv_rank=16, kinds=("moe", "dense"), experts=4, identity=0,
                  groups=None, top=1, shared_ff=0, side_dim=0, bigram=None, emb_scale=1.0),
    # head sizes that tile into 16s (the tensor-core attention of a 16-bit model), all experts in one kept group of two, a side
    # input as wide as a head
    "tile": dict(width=64, vocab=83, heads=4, dim=32, vdim=16, q_rank=24, kv_rank=64, kinds=("moe", "moe", "dense"), experts=6,
                 identity=2, groups=(2, 1), top=4, expert_ff=24, shared_ff=8, side_dim=16, bigram=(7, 5, 3)),
    # head sizes and ranks that tile into nothing (24, 40, 100, 12), five heads, sixteen experts in four groups of which two are
    # kept, no identity experts, a layer without feed-forward first, a side input of three channels
    "wide": dict(width=72, vocab=300, heads=5, dim=24, vdim=40, q_rank=12, kv_rank=100, scale=0.15, ff=56, kinds=(None, "moe", "dense", "moe"),
                 experts=16, identity=0, groups=(4, 2), top=3, expert_ff=8, shared_ff=40, side_dim=3, bigram=(211, 3, 1000003), emb_scale=1.3),
    # no side input while the depth average is on: a layer's last addition is then the feed-forward's, or the mixer's own
    "bare": dict(width=40, vocab=50, heads=4, dim=16, vdim=32, q_rank=16, kv_rank=128, kinds=(None, "dense", None), side_dim=0, bigram=(17, 1, 1)),
}
OPTIONS = {"plain": dict(layer_scale=False, depth_average=False), "bare": dict(layer_scale=False)}


def make(name, seed=0):
    cfg = O.random_config(**CONFIGS[name])
    w = O.random_weights(cfg, seed + 1, **OPTIONS.get(name, {}))
    return cfg, w


def w64(w):
    return {k: v.to(F64) for k, v in w.items()}


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


# ================================================================== CPU: configuration, loader, cache bookkeeping
def test_loader_maps_every_tensor_and_merges(tmp_path):
    from ipex_llm_b200.transformers.models.utils import read_safetensors
    cfg, w = make("odd")
    save_checkpoint(cfg, w, tmp_path)
    back = read_safetensors(os.path.join(tmp_path, "model.safetensors"))
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    model = load_framework(tmp_path, torch.bfloat16)
    assert type(model).__name__ == "SerotarForCausalLM" and model.config.model_type == "serotar"
    assert model.config.layer_scale and model.config.depth_average
    mx = model.model.layers[0].mixer
    assert mx.in_proj.weight.shape == (20 + 22, cfg["width"]) and not hasattr(mx, "dq")
    assert torch.equal(mx.in_proj.weight[:20], w["l0.mix.dq"]) and torch.equal(mx.in_proj.weight[20:], w["l0.mix.dkv"])
    assert torch.equal(mx.expand.weight[:3 * 8], w["l0.mix.uk"]) and torch.equal(mx.expand.weight[3 * 8:], w["l0.mix.uv"])
    moe = model.model.layers[1].mlp
    assert (moe.n_experts, moe.n_identity, moe.n_out, moe.groups, moe.keep, moe.top) == (6, 3, 9, 3, 2, 3)
    assert torch.equal(moe.experts[4].gate_up.weight, torch.cat([w["l1.mlp.e4.gate"], w["l1.mlp.e4.up"]]))
    assert torch.equal(moe.shared.down.weight, w["l1.mlp.shared.down"])
    assert model.model.layers[2].mlp is None and model.model.layers[2].dwa.shape == (4,)
    assert model.model.norm.weight.shape == () and model.model.pair_embed.weight.shape == (54, cfg["width"])
    # what the checkpoint does not have does not exist in the model either
    cfg2, w2 = make("plain")
    save_checkpoint(cfg2, w2, tmp_path / "plain")
    plain = load_framework(tmp_path / "plain", torch.float32)
    assert plain.model.pair_embed is None and plain.model.side_embed is None and plain.model.layers[0].ls1 is None
    assert plain.model.layers[0].dwa is None and plain.model.layers[0].mlp.shared is None and plain.model.layers[0].mlp.groups == 1
    assert not plain.config.layer_scale and not plain.config.depth_average
    # a tensor of the wrong shape is refused, by name
    bad = dict(w)
    bad["l1.mlp.correction"] = torch.zeros(4, dtype=torch.bfloat16)
    save_checkpoint(cfg, bad, tmp_path / "bad")
    with pytest.raises(RuntimeError, match="correction"):
        load_framework(tmp_path / "bad", torch.bfloat16)


def test_registry_picks_the_design(tmp_path):
    from ipex_llm_b200.transformers.model import native_architecture
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Serotar"}))
    assert native_architecture(tmp_path).endswith("models.serotar")


def test_latent_cache_bookkeeping():
    from ipex_llm_b200.transformers import kv
    cache = kv.DynamicStateCache()
    cache.start(torch.tensor([[0, 1, 1], [1, 1, 1], [0, 0, 1]]), 3, 3, torch.device("cpu"))
    lat = cache.run_state(1, latent=True).kv
    assert isinstance(lat, kv.LatentKVLayer)
    store, held = lat.slots(3, 5, 3, torch.float32, torch.device("cpu"))
    assert held == 0 and store.shape == (3, lat.capacity(), 5) and lat.capacity() >= 3
    store[:, :3] = torch.arange(3.0)[:, None, None] * 10 + torch.arange(3.0)[None, :, None]
    lat.commit(3)
    prev = cache.previous_tokens(3, torch.device("cpu"))
    prev.copy_(torch.tensor([7, 8, 9]))
    cache.advance(3)
    old_block, kv.KV_ALLOC_BLOCK_LENGTH = kv.KV_ALLOC_BLOCK_LENGTH, 2
    try:
        first_store = lat.store
        store, held = lat.slots(3, 5, lat.capacity(), torch.float32, torch.device("cpu"))       # more than is free: the storage moves
        assert held == 3 and store is not first_store and torch.equal(store[:, :3], first_store[:, :3])
    finally:
        kv.KV_ALLOC_BLOCK_LENGTH = old_block
    cache.batch_select_indices([2, 0])
    assert cache.pad.tolist() == [2, 1] and cache.previous_tokens(2, torch.device("cpu")).tolist() == [9, 7]
    assert lat.held()[:, :, 0].tolist() == [[20.0, 21.0, 22.0], [0.0, 1.0, 2.0]] and lat.get_seq_length() == 3
    address = lat.store.data_ptr()
    cache.restart()
    assert lat.get_seq_length() == 0 and lat.store.data_ptr() == address and cache.seen == 0


def test_oracle_router_against_brute_force():
    g = torch.Generator().manual_seed(5)
    h, router = torch.randn(40, 12, generator=g, dtype=F64), torch.randn(12, 12, generator=g, dtype=F64)
    corr = torch.randn(12, generator=g, dtype=F64) * 0.1 - 3.0            # all choice scores negative
    r = {"experts": 10, "identity": 2, "top": 3, "groups": {"count": 4, "keep": 2}}
    chosen, weights = O.route(h, router, corr, r)
    for t in range(40):
        s = torch.softmax(router @ h[t], 0)
        c = (s + corr).tolist()
        gs = sorted(range(4), key=lambda k: -max(c[3 * k:3 * k + 3]))[:2]
        allowed = [e for e in range(12) if e // 3 in gs]
        want = sorted(allowed, key=lambda e: -c[e])[:3]
        assert sorted(chosen[t].tolist()) == sorted(want)
        assert torch.allclose(weights[t], s[chosen[t]])


# ================================================================== GPU: each mechanism alone
@pytest.fixture(scope="module")
def mixers(cuda_device):
    from ipex_llm_b200.transformers.models import mixer_ops
    return mixer_ops


def _rand(shape, gen, dtype, device, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype).to(device)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(2)
    V, W, buckets, mp, mc = 37, 19, 11, 1000003, 77
    table, pair = _rand((V, W), g, dtype, cuda_device), _rand((buckets + 1, W), g, dtype, cuda_device)
    seqs = [tokens_for({"vocab": V}, n, 10 + n) for n in (9, 4, 6)]
    pad = torch.tensor([0, 5, 3], dtype=torch.int32, device=cuda_device)
    ids = torch.zeros(3, 9, dtype=torch.int64)
    for b, s in enumerate(seqs):
        ids[b, 9 - len(s):] = torch.tensor(s)
    ids = ids.to(cuda_device)
    want = [O.embedding(s, table.cpu().to(F64), 0.37, pair.cpu().to(F64), buckets, mp, mc) for s in seqs]
    # the first five slots, then the rest: the pair of slot 5 needs the token of slot 4 from the state
    prev = torch.zeros(3, dtype=torch.int64, device=cuda_device)
    copy = torch.empty(15, W, dtype=torch.float32, device=cuda_device)
    x1, h1 = mixers.embed_pair(table, 0.37, pair, buckets, mp, mc, ids[:, :5].contiguous(), prev, 0, pad, dtype, x_copy=copy)
    prev.copy_(ids[:, 4])
    x2, _ = mixers.embed_pair(table, 0.37, pair, buckets, mp, mc, ids[:, 5:].contiguous(), prev, 5, pad, dtype)
    x2b, _ = mixers.embed_pair(table, 0.37, pair, buckets, mp, mc, ids[:, 6:].contiguous(), ids[:, 5].contiguous(), 1, None, dtype)
    assert torch.equal(x2b.view(3, 3, W), x2.view(3, 4, W)[:, 1:])          # later calls need neither padding nor the slot number
    x = torch.cat([x1.view(3, 5, W), x2.view(3, 4, W)], 1).cpu().to(F64)
    assert torch.equal(copy, x1) and (h1.float() - x1).abs().max() <= (0.0 if dtype == torch.float32 else 0.05)
    for b, s in enumerate(seqs):
        assert (x[b, 9 - len(s):] - want[b]).abs().max() < 1e-5
        assert x[b, :9 - len(s)].abs().sum() == 0                        # padding
    # no pair table at all
    x3, _ = mixers.embed_pair(table, 2.0, None, 0, 0, 0, ids, prev, 0, torch.zeros(3, dtype=torch.int32, device=cuda_device), dtype)
    assert (x3.cpu().to(F64) - 2.0 * table.cpu().to(F64)[ids.cpu().reshape(-1)]).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,n", [(45, 5), (1100, 5), (8200, 3), (40, 1100)])
def test_residual_norm_and_depth_average(mixers, cuda_device, dtype, width, n):
    """rows held in registers (few rows, up to 8192 wide) and the plain loop (wider rows; many rows under a depth average)"""
    g = torch.Generator().manual_seed(4)
    eps = 1e-3
    x0 = torch.randn(n, width, generator=g)
    gain, vec = _rand((), g, dtype, cuda_device) + 1.5, _rand((width,), g, dtype, cuda_device)
    coef = _rand((3,), g, dtype, cuda_device)
    stack = torch.randn(4, n, width, generator=g).to(cuda_device)
    for y in (_rand((n, width), g, dtype, cuda_device, 3.0), _rand((n, width), g, torch.float32, cuda_device, 3.0)):
        ny = O.rms(y.cpu().to(F64), eps)
        x = x0.clone().to(cuda_device)
        h = mixers.rms_residual(x, y, gain, vec, eps, dtype)
        want = x0.to(F64) + ny * gain.cpu().to(F64) * vec.cpu().to(F64)
        assert (x.cpu().to(F64) - want).abs().max() < 2e-5 and (h.cpu().to(F64) - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.1)
        x = x0.clone().to(cuda_device)
        mixers.rms_residual(x, y, None, vec, eps, dtype, want_h=False)
        assert (x.cpu().to(F64) - (x0.to(F64) + ny * vec.cpu().to(F64))).abs().max() < 2e-5
        # kept as stream 2, then the weighted sum of streams 0..2
        x = x0.clone().to(cuda_device)
        st = stack.clone()
        mixers.rms_residual(x, y, gain, None, eps, dtype, stack=st, index=2, coef=coef)
        new = x0.to(F64) + ny * gain.cpu().to(F64)
        assert (st[2].cpu().to(F64) - new).abs().max() < 2e-5 and torch.equal(st[3], stack[3]) and torch.equal(st[:2], stack[:2])
        c = coef.cpu().to(F64)
        want = c[0] * stack[0].cpu().to(F64) + c[1] * stack[1].cpu().to(F64) + c[2] * new
        assert (x.cpu().to(F64) - want).abs().max() < 3e-5
    xn = mixers.rms_norm_rows(x0.to(cuda_device), gain, None, eps, dtype)
    assert (xn.cpu().to(F64) - O.rms(x0.to(F64), eps) * gain.cpu().to(F64)).abs().max() < (2e-5 if dtype == torch.float32 else 0.05)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(6)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    z = _rand((11, 37), g, dtype, cuda_device, 2.0)
    pq = torch.tensor([0.3, -1.2]).to(dtype).to(cuda_device)
    want = O.xielu(z.cpu().to(F64), pq.cpu().to(F64)[0], pq.cpu().to(F64)[1])
    got = mixers.xielu(z, pq).cpu().to(F64)
    assert ((got - want).abs() / (1 + want.abs())).max() < tol
    assert (z <= 0).any() and (z > 0).any()
    gu = _rand((7, 26), g, dtype, cuda_device, 2.0)
    want = O.silu(gu.cpu().to(F64)[:, :13]) * gu.cpu().to(F64)[:, 13:]
    assert ((mixers.silu_mul(gu, 13).cpu().to(F64) - want).abs() / (1 + want.abs())).max() < tol
    table, ids = _rand((9, 20), g, dtype, cuda_device), torch.tensor([3, 0, 8, 8, 1, 2, 5], device=cuda_device)
    gate = _rand((7, 5), g, dtype, cuda_device, 2.0)
    want = O.gelu_tanh(gate.cpu().to(F64)) * table.cpu().to(F64)[ids.cpu()][:, 10:15]
    assert ((mixers.gelu_table_mul(gate, table, 10, ids).cpu().to(F64) - want).abs() / (1 + want.abs())).max() < tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(7)
    B, S, qr, kr, held, cap, eps = 2, 3, 10, (13 if dtype == torch.float32 else 1100), 4, 9, 1e-4       # 1100: wider than the registers hold
    proj = _rand((B, S, 2 + qr + 3 + kr), g, dtype, cuda_device, 2.0)
    qw, cw = _rand((qr,), g, dtype, cuda_device), _rand((kr,), g, dtype, cuda_device)
    store = torch.full((B, cap, kr), 9.0, dtype=dtype, device=cuda_device)
    pad = torch.tensor([0, 6], dtype=torch.int32, device=cuda_device)       # row 1: slots 4, 5 are padding, slot 6 is its first token
    cq = mixers.latent_prepare(proj, 2, qr, qw, 2 + qr + 3, kr, cw, eps, store, held, 0, pad)
    p = proj.cpu().to(F64)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    want_q = O.rms(p[..., 2:2 + qr], eps) * qw.cpu().to(F64)
    want_c = O.rms(p[..., 2 + qr + 3:], eps) * cw.cpu().to(F64)
    assert (cq.view(B, S, qr)[0].cpu().to(F64) - want_q[0]).abs().max() < tol
    assert (store[0, held:held + S].cpu().to(F64) - want_c[0]).abs().max() < tol
    assert store[1, held:held + 2].abs().max() == 0 and (store[1, held + 2].cpu().to(F64) - want_c[1, 2]).abs().max() < tol
    assert (store[:, :held] == 9).all() and (store[:, held + S:] == 9).all()


def _attention_case(g, B, S, held, H, G, D, Dv, dtype, device, extra=3):
    """random q and keys / values that live inside wider tensors (strides larger than the head sizes)"""
    L = held + S
    q = _rand((B * S, H * D), g, dtype, device)
    kfull, vfull = _rand((B, L + extra, G, D + 8), g, dtype, device), _rand((B, L + extra, G, Dv + 16), g, dtype, device)
    return q, kfull[..., 8:], vfull[..., :Dv]


def _attention_want(q, k, v, B, S, held, H, scale, window, pads):
    D = k.shape[3]
    out = []
    for b in range(B):
        qb = q.view(B, S, H, D)[b].cpu().to(F64)
        out.append(O.windowed_attention(qb, k[b].cpu().to(F64), v[b].cpu().to(F64), scale, window, pads[b], held).reshape(S, -1))
    return torch.stack(out).reshape(B * S, -1)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S,held,H,G,D,Dv,window", [
    (torch.float32, 5, 0, 6, 2, 5, 7, 0), (torch.float32, 1, 300, 4, 1, 24, 600, 0), (torch.float32, 3, 40, 2, 2, 16, 16, 7),
    (torch.bfloat16, 1, 517, 3, 1, 64, 64, 0), (torch.bfloat16, 4, 30, 4, 2, 10, 6, 0), (torch.float32, 70, 3, 2, 1, 9, 33, 20)])
def test_softmax_attention_general(mixers, cuda_device, dtype, S, held, H, G, D, Dv, window):
    g = torch.Generator().manual_seed(S * 100 + held)
    B = 2
    q, k, v = _attention_case(g, B, S, held, H, G, D, Dv, dtype, cuda_device)
    pads = [0, min(held + S - 1, 3)]
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    got = mixers.softmax_attention(q, k, v, B, S, H, held, 0, pad, window, 0.4, tensor_cores=False)
    want = _attention_want(q, k, v, B, S, held, H, 0.4, window, pads)
    assert (got.cpu().to(F64) - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.02)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,held,H,G,D,Dv,window", [(16, 0, 2, 2, 16, 16, 0), (150, 0, 3, 1, 32, 48, 0), (70, 200, 4, 2, 64, 128, 0),
                                                      (33, 31, 2, 1, 128, 32, 0), (100, 60, 2, 2, 256, 16, 40), (64, 0, 1, 1, 16, 256, 0)])
def test_softmax_attention_tensor_cores(mixers, cuda_device, dtype, S, held, H, G, D, Dv, window):
    g = torch.Generator().manual_seed(S + held)
    B = 2
    q, k, v = _attention_case(g, B, S, held, H, G, D, Dv, dtype, cuda_device, extra=0)
    pads = [0, min(held + S - 1, 37)]
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    scale = 2.0 / D ** 0.5
    got = mixers.softmax_attention(q, k, v, B, S, H, held, 0, pad, window, scale, tensor_cores=True)
    same = mixers.softmax_attention(q, k, v, B, S, H, held, 0, pad, window, scale, tensor_cores=False)
    want = _attention_want(q, k, v, B, S, held, H, scale, window, pads)
    assert (got.cpu().to(F64) - want).abs().max() < 0.02 and (same.cpu().to(F64) - want).abs().max() < 0.02
    # the weights carry more than the 8 bits of a rounded 16-bit number: the two kernels agree far below that
    assert (got.float() - same.float()).abs().max() < 0.012


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S", [(torch.float32, 1), (torch.float32, 40), (torch.bfloat16, 1), (torch.bfloat16, 40)])
def test_one_outstanding_key_decides(mixers, cuda_device, dtype, S):
    """a key whose score dwarfs all others: the output is its value when it is visible and must not show it otherwise -- far
    back among hundreds, just inside and just outside a window, at the borders of the kernels' key tiles, in front of a row's
    first token, and in the future"""
    g = torch.Generator().manual_seed(11)
    H, D, Dv, L = 2, 16, 16, 700
    held = L - S
    base_k, base_v = torch.randn(1, L + 8, 1, D, generator=g) * 0.1, torch.randn(1, L + 8, 1, Dv, generator=g)
    q = torch.randn(S, H * D, generator=g) * 0.1
    spike = torch.zeros(D)
    spike[3] = 40.0
    q = q + spike.repeat(H)[None] * 0.05                                   # q . spike key = 80 + noise

    def run(at, window, first=0, tc=False):
        k = base_k.clone()
        k[0, at, 0] = spike
        out = mixers.softmax_attention(q.to(dtype).to(cuda_device), k.to(dtype).to(cuda_device), base_v.to(dtype).to(cuda_device), 1, S, H, held, 0,
                                       torch.tensor([first], dtype=torch.int32, device=cuda_device), window, 1.0, tensor_cores=tc)
        return out.float().cpu().view(S, H, Dv)

    last = S - 1                                                            # the last query sits at storage index L - 1
    for tc in ([False, True] if (dtype != torch.float32 and S >= 16) else [False]):
        for at in (0, 1, 31, 32, 63, 64, 255, 256, 257, L - 2, L - 1):      # visible to the last query wherever it is
            assert (run(at, 0, tc=tc)[last] - base_v[0, at, 0]).abs().max() < 0.02, at
        # a window of 100: index L - 100 is the oldest visible one
        assert (run(L - 100, 100, tc=tc)[last] - base_v[0, L - 100, 0]).abs().max() < 0.02
        assert (run(L - 101, 100, tc=tc)[last] - base_v[0, L - 101, 0]).abs().max() > 0.3
        # in front of the row's first token (padding), and the row's first token itself
        assert (run(4, 0, first=5, tc=tc)[last] - base_v[0, 4, 0]).abs().max() > 0.3
        assert (run(5, 0, first=5, tc=tc)[last] - base_v[0, 5, 0]).abs().max() < 0.02
        # the future: a key behind the last query, and for several new tokens a key that only the later ones may see
        assert (run(L, 0, tc=tc)[last] - base_v[0, L, 0]).abs().max() > 0.3
        if S > 1:
            out = run(held + 20, 0, tc=tc)
            assert (out[20] - base_v[0, held + 20, 0]).abs().max() < 0.02 and (out[19] - base_v[0, held + 20, 0]).abs().max() > 0.3


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,held,H,G,D,Dv,window,latent", [(1, 700, 16, 1, 512, 512, 0, True), (1, 63, 8, 2, 64, 128, 0, False),
                                                             (3, 130, 4, 1, 32, 256, 0, False), (16, 200, 6, 1, 128, 128, 0, True),
                                                             (2, 300, 8, 2, 48, 128, 90, False), (1, 0, 4, 1, 256, 256, 0, True)])
def test_softmax_attention_shared_heads(mixers, cuda_device, dtype, S, held, H, G, D, Dv, window, latent):
    """few new tokens whose heads share keys and values: one pass over the keys for all heads, key ranges split over blocks and
    merged; ``latent``: keys and values are the same tensor (a latent cache read as one shared head)"""
    g = torch.Generator().manual_seed(S * 7 + held)
    B = 3
    q, k, v = _attention_case(g, B, S, held, H, G, D, Dv, dtype, cuda_device, extra=5)
    q = q * 0.5
    if latent:
        v = k
    pads = [0, min(held + S - 1, 41), 0]
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    scale = 1.5 / D ** 0.5
    from ipex_llm_b200.ggml.model import mixers_cpp
    assert mixers_cpp.lib().mixers_softmax_attention_workspace(mixers_cpp.dtype_code(dtype), B, S, H, G, D, Dv) > 0
    got = mixers.softmax_attention(q, k, v, B, S, H, held, 0, pad, window, scale, tensor_cores=True)
    same = mixers.softmax_attention(q, k, v, B, S, H, held, 0, pad, window, scale, tensor_cores=False)
    want = _attention_want(q, k, v, B, S, held, H, scale, window, pads)
    assert (got.cpu().to(F64) - want).abs().max() < 0.02 and (same.cpu().to(F64) - want).abs().max() < 0.02
    assert (got.float() - same.float()).abs().max() < 0.012
    # the length read from the device, as a replayed step does
    dyn = torch.tensor([held], dtype=torch.int32, device=cuda_device)
    again = mixers.softmax_attention(q, k, v, B, S, H, 0, 0, pad, window, scale, dyn=dyn, tensor_cores=True)
    assert torch.equal(again, got)


@pytest.mark.gpu
def test_one_outstanding_key_decides_for_shared_heads(mixers, cuda_device):
    """the same proof for the kernel that splits the keys over blocks: a far key, the borders of its 64-key tiles and of its
    key ranges, a window's two sides, padding, the future"""
    g = torch.Generator().manual_seed(12)
    H, D, L = 8, 128, 1500
    base = torch.randn(1, L + 8, 1, D, generator=g) * 0.1
    spike = torch.zeros(D)
    spike[5] = 3.0
    q = (torch.randn(1, H * D, generator=g) * 0.1 + spike.repeat(H)[None] * 8).to(torch.bfloat16).to(cuda_device)      # q . spike = 72

    def run(at, window=0, first=0):
        c = base.clone()
        c[0, at, 0] = spike
        c = c.to(torch.bfloat16).to(cuda_device)
        out = mixers.softmax_attention(q, c, c, 1, 1, H, L - 1, 0, torch.tensor([first], dtype=torch.int32, device=cuda_device), window, 1.0)
        return out.float().cpu().view(H, D)

    for at in (0, 63, 64, 127, 128, 191, 192, 700, 1023, 1024, L - 2, L - 1):
        assert (run(at) - spike).abs().max() < 0.05, at
    assert (run(L - 200, window=200) - spike).abs().max() < 0.05 and (run(L - 201, window=200) - spike).abs().max() > 1.0
    assert (run(9, first=10) - spike).abs().max() > 1.0 and (run(10, first=10) - spike).abs().max() < 0.05
    assert (run(L) - spike).abs().max() > 1.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_out,groups,keep,top,shift", [(9, 3, 2, 3, 0.0), (12, 4, 2, 3, -3.0), (8, 1, 1, 8, 0.0), (10, 10, 3, 3, 0.0),
                                                           (64, 8, 4, 6, -1.0), (5, 1, 1, 1, 0.0), (6, 3, 1, 2, 0.0)])
def test_grouped_router(mixers, cuda_device, dtype, n_out, groups, keep, top, shift):
    g = torch.Generator().manual_seed(n_out)
    n, w = 50, 37
    h, router = _rand((n, w), g, dtype, cuda_device), _rand((n_out, w), g, dtype, cuda_device, 0.4)
    corr = (_rand((n_out,), g, dtype, cuda_device, 0.2) + shift).to(dtype)  # shift < 0: every choice score is negative
    idx, wgt = mixers.grouped_router(h, router, corr, groups, keep, top)
    r = {"top": top, "groups": {"count": groups, "keep": keep}}
    chosen, weights = O.route(h.cpu().to(F64), router.cpu().to(F64), corr.cpu().to(F64), r)
    assert torch.equal(idx.cpu().to(torch.int64).sort(1).values, chosen.sort(1).values)
    got = torch.zeros(n, n_out, dtype=F64).scatter_(1, idx.cpu().to(torch.int64), wgt.cpu().to(F64))
    want = torch.zeros(n, n_out, dtype=F64).scatter_(1, chosen, weights)
    assert (got - want).abs().max() < 1e-5                                  # the router is 32-bit whatever the dtype


@pytest.mark.gpu
@pytest.mark.parametrize("n,top,n_keys", [(1, 1, 2), (37, 3, 10), (5000, 4, 65), (300, 2, 1025)])
def test_pairs_sorted_by_expert(mixers, cuda_device, n, top, n_keys):
    g = torch.Generator().manual_seed(n)
    idx = torch.randint(0, n_keys, (n, top), generator=g).to(torch.int32).to(cuda_device)
    counts, pos, token_of = mixers.moe_sort(idx, n_keys)
    flat = idx.reshape(-1).cpu().to(torch.int64)
    assert torch.equal(counts.cpu().to(torch.int64), torch.bincount(flat, minlength=n_keys))
    p = pos.reshape(-1).cpu().to(torch.int64)
    assert torch.equal(p.sort().values, torch.arange(n * top))                                # a permutation
    assert torch.equal(token_of.cpu()[p], torch.arange(n * top) // top)                       # every row knows its token
    by_row = torch.empty(n * top, dtype=torch.int64)
    by_row[p] = flat
    assert torch.equal(by_row, flat.sort().values)                                            # rows are grouped by output, in order


# ================================================================== GPU: the model
def build(tmp_path, name, dtype, device, seed=0, **kw):
    cfg, w = make(name, seed)
    folder = tmp_path / f"{name}{seed}"
    save_checkpoint(cfg, w, folder)
    return cfg, w64(w), load_framework(folder, dtype, device, **kw)


@torch.no_grad()
def run_portions(model, tokens, sizes, device):
    """one request fed in portions (the last size repeats); returns logits [T, V]"""
    ids = torch.tensor([tokens], device=device)
    cache, out, at, i = None, [], 0, 0
    while at < len(tokens):
        n = sizes[min(i, len(sizes) - 1)]
        o = model(input_ids=ids[:, at:at + n], past_key_values=cache, use_cache=True)
        cache = o.past_key_values
        out.append(o.logits[0])
        at, i = at + n, i + 1
    return torch.cat(out)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_decode_and_portions_against_the_oracle(tmp_path, cuda_device, name, dtype):
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    tokens = tokens_for(cfg, 75, 3)
    collect = []
    want = O.forward(cfg, w, tokens, collect)
    model.collect_residual = []
    whole = run_portions(model, tokens, [len(tokens)], cuda_device)
    if dtype == torch.float32:                                              # the stream after every layer, too
        for got, ref in zip(model.collect_residual, collect):
            assert (got[0].cpu().to(F64) - ref).abs().max() < 1e-4 * max(1.0, ref.abs().max())
    model.collect_residual = None
    assert_close(whole, want, dtype)
    assert_close(run_portions(model, tokens, [40, 1], cuda_device), want, dtype)            # a prompt, then token by token
    assert_close(run_portions(model, tokens, [1], cuda_device), want, dtype)                # from the first token on
    for sizes in ([2], [3, 17, 2, 30], [20, 20, 19, 16], [1, 1, 40, 2]):
        assert_close(run_portions(model, tokens, sizes, cuda_device), want, dtype)
    if dtype != torch.float32:                                              # the general attention kernel under a 16-bit model
        model.attention_tensor_cores = False
        assert_close(run_portions(model, tokens, [len(tokens)], cuda_device), want, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_few_tokens_and_many_tokens_agree(tmp_path, cuda_device, dtype):
    """the host-free path (address tables) and the sorted path compute the same layer; both match the plain statement"""
    from ipex_llm_b200.transformers.models import serotar
    cfg, w, model = build(tmp_path, "odd", dtype, cuda_device)
    mlp, spec = model.model.layers[1].mlp, cfg["layers"][1]["mlp"]
    g = torch.Generator().manual_seed(8)
    h = _rand((20, cfg["width"]), g, dtype, cuda_device)
    want = O.moe_ff(h.cpu().to(F64), O.sub(w, "l1.mlp."), spec)
    few = model._experts(mlp, h, False)
    old, serotar.MOE_SMALL_TOKENS = serotar.MOE_SMALL_TOKENS, 0
    try:
        many = model._experts(mlp, h, False)
    finally:
        serotar.MOE_SMALL_TOKENS = old
    tol = 2e-5 if dtype == torch.float32 else 0.06
    assert few.dtype == torch.float32 and (few.cpu().to(F64) - want).abs().max() < tol and (many.cpu().to(F64) - want).abs().max() < tol
    assert (few - many).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)
    # a token whose choices are all identity experts: its output is the input times the weights (+ the shared expert)
    mlp.correction.data[6:] = 5.0
    idx, wgt = serotar.ops.grouped_router(h, mlp.router, mlp.correction, mlp.groups, mlp.keep, mlp.top)
    assert (idx >= 6).all()
    w2 = dict(O.sub(w, "l1.mlp."))
    w2["correction"] = mlp.correction.detach().cpu().to(F64)
    want = O.moe_ff(h.cpu().to(F64), w2, spec)
    for limit in (serotar.MOE_SMALL_TOKENS, 0):
        old, serotar.MOE_SMALL_TOKENS = serotar.MOE_SMALL_TOKENS, limit
        try:
            assert (model._experts(mlp, h, False).cpu().to(F64) - want).abs().max() < tol
        finally:
            serotar.MOE_SMALL_TOKENS = old


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "tile"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_matches_each_request_alone(tmp_path, cuda_device, name, dtype):
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    lens, extra = [1, 23, 50, 7], 6
    seqs = [tokens_for(cfg, n + extra, 20 + n) for n in lens]
    want = [O.forward(cfg, w, s) for s in seqs]
    width = max(lens)
    ids = torch.zeros(4, width, dtype=torch.int64)
    mask = torch.zeros(4, width, dtype=torch.int64)
    for b, (s, n) in enumerate(zip(seqs, lens)):
        ids[b, width - n:] = torch.tensor(s[:n])
        mask[b, width - n:] = 1
    with torch.no_grad():
        o = model(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), use_cache=True)
        cache = o.past_key_values
        for b, n in enumerate(lens):
            assert_close(o.logits[b, width - n:], want[b][:n], dtype)
        rows = [0, 1, 2, 3]
        for step in range(extra):
            if step == 2:                                                   # two requests end: their rows leave the batch
                cache.batch_select_indices(torch.tensor([3, 1]))
                rows = [3, 1]
            nxt = torch.tensor([[seqs[b][lens[b] + step]] for b in rows], device=cuda_device)
            o = model(input_ids=nxt, past_key_values=cache, use_cache=True)
            for r, b in enumerate(rows):
                assert_close(o.logits[r], want[b][lens[b] + step:lens[b] + step + 1], dtype)


@pytest.mark.gpu
def test_long_decoding_through_growing_storage(tmp_path, cuda_device):
    """300 tokens one by one from a 5-token prompt: the latent cache outgrows its first block and moves"""
    cfg, w, model = build(tmp_path, "tile", torch.float32, cuda_device)
    tokens = tokens_for(cfg, 305, 9)
    want = O.forward(cfg, w, tokens)
    got = run_portions(model, tokens, [5, 1], cuda_device)
    assert_close(got, want, torch.float32)
    # a far token decides: the prompt's second token is repeated nowhere else, so its pair and its latent are unique
    assert position_errors(got[-1:], want[-1:]).max() < 3e-5


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "plain"])
def test_greedy_generate_matches_the_oracle(tmp_path, cuda_device, monkeypatch, name):
    cfg, w, model = build(tmp_path, name, torch.float32, cuda_device)
    prompt = tokens_for(cfg, 9, 4)
    want = O.greedy(cfg, w, prompt, 12)
    ids = torch.tensor([prompt], device=cuda_device)
    got = model.generate(ids, max_new_tokens=12, do_sample=False)
    assert model.__dict__.get("_b200_state_graph_failed") is None and model.__dict__.get("_b200_state_graphs")     # the recorded step ran
    assert got[0].tolist() == want
    # the step's cache serves other requests afterwards: a batch of two with padding, then the first request again
    other = tokens_for(cfg, 4, 5)
    want2 = O.greedy(cfg, w, other, 7)
    batch = torch.tensor([prompt, [0] * 5 + other], device=cuda_device)
    mask = torch.tensor([[1] * 9, [0] * 5 + [1] * 4], device=cuda_device)
    got2 = model.generate(batch, attention_mask=mask, max_new_tokens=7, do_sample=False)
    assert got2[0].tolist() == want[:16] and got2[1, 5:].tolist() == want2
    assert model.generate(ids, max_new_tokens=12, do_sample=False)[0].tolist() == want
    # transformers' own loop on the same forward
    monkeypatch.setenv("IPEX_LLM_B200_DECODE_GRAPH", "0")
    assert model.generate(ids, max_new_tokens=12, do_sample=False)[0].tolist() == want


@pytest.mark.gpu
def test_recorded_step_of_a_16_bit_model_equals_the_eager_loop(tmp_path, cuda_device, monkeypatch):
    """a bf16 model whose decoding attention is the one-pass kernel over the latent cache (4 heads on a latent of 128): the
    replayed step reads the cache length from the device and must produce the tokens of the loop that passes it from the host"""
    cfg, w, model = build(tmp_path, "bare", torch.bfloat16, cuda_device)
    prompts = torch.tensor([tokens_for(cfg, 70, 1), [0] * 30 + tokens_for(cfg, 40, 2)], device=cuda_device)
    mask = torch.tensor([[1] * 70, [0] * 30 + [1] * 40], device=cuda_device)
    replayed = model.generate(prompts, attention_mask=mask, max_new_tokens=80, do_sample=False)
    assert model.__dict__.get("_b200_state_graph_failed") is None and model.__dict__.get("_b200_state_graphs")
    monkeypatch.setenv("IPEX_LLM_B200_DECODE_GRAPH", "0")
    eager = model.generate(prompts, attention_mask=mask, max_new_tokens=80, do_sample=False)
    assert torch.equal(replayed, eager)
    # and both follow the plain statement as far as a 16-bit model can: the first new token of each row
    for b, n in ((0, 70), (1, 40)):
        want = O.forward(cfg, w, prompts[b, 70 - n:].tolist())[-1]
        top2 = want.topk(2).values
        if top2[0] - top2[1] > 0.5:
            assert int(replayed[b, 70]) == int(want.argmax())


@pytest.mark.gpu
def test_low_bit_conversion_runs_the_same_model(tmp_path, cuda_device, native_lib):
    """the projections are ordinary linears to the converter: a sym_int4 model answers close to the 16-bit one, its experts
    (no longer plain matrices) take the sorted path also for one token"""
    from ipex_llm_b200.transformers.low_bit_linear import LowBitLinear
    cfg = O.random_config(width=128, vocab=90, heads=2, dim=32, vdim=32, q_rank=64, kv_rank=64, ff=128, kinds=("moe", "dense"), experts=4,
                          identity=1, groups=None, top=2, expert_ff=64, shared_ff=64, side_dim=0)
    w = O.random_weights(cfg, 3)
    save_checkpoint(cfg, w, tmp_path / "m")
    ref = load_framework(tmp_path / "m", torch.bfloat16, cuda_device)
    low = load_framework(tmp_path / "m", torch.bfloat16, None, load_in_low_bit="sym_int4").to(cuda_device)
    assert isinstance(low.model.layers[0].mixer.in_proj, LowBitLinear) and isinstance(low.model.layers[0].mlp.experts[0].down, LowBitLinear)
    assert low.model.layers[0].mlp.address_tables(torch.bfloat16, cuda_device) is None
    tokens = tokens_for(cfg, 30, 1)
    a = run_portions(ref, tokens, [30], cuda_device)
    b = run_portions(low, tokens, [25, 1], cuda_device)
    assert torch.isfinite(b).all() and position_errors(b, a.cpu().to(F64)).quantile(0.8) < 0.5
