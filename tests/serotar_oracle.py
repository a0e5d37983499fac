"""Plain statements of the Serotar design's mechanisms (PyTorch, any dtype; the tests use float64), one function each, and a
whole-model forward that recomputes every position from the full token list.  Nothing here is shared with the package:
weights come in as a dict of tensors under the checkpoint's names, the configuration as the parsed config.json.
"""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0)


def xielu(z, p, q):
    """quadratic branch a z^2 + z/2 (a = softplus(p)) for positive z, exponential branch c (expm1(z) - z) + z/2 (c = 1/2 + softplus(q)) otherwise"""
    ap, aq = softplus(p), 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    zn = z.clamp(max=0)
    neg = aq * (torch.expm1(zn) - zn) + 0.5 * zn
    return torch.where(z > 0, pos, neg)


def silu(z):
    return z * torch.sigmoid(z)


def embedding(tokens, embed, scale, bigram=None, buckets=0, mul_prev=0, mul_cur=0):
    """tokens: list of ints of ONE sequence.  Row of the bigram table: (previous * mul_prev + current * mul_cur) mod buckets,
    row number ``buckets`` for the first token."""
    t = torch.tensor(tokens, dtype=torch.int64)
    x = embed[t] * scale
    if bigram is not None:
        rows = [buckets] + [(tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets for i in range(1, len(tokens))]
        x = x + bigram[torch.tensor(rows, dtype=torch.int64)]
    return x


def scalar_norm(y, g, eps):
    """RMS norm with a single gain"""
    return rms(y, eps) * g


def latent_attention(h, W, m, eps):
    """h [T, width] of one sequence.  W: the mixer's tensors by short name (dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o)."""
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    cq = rms(h @ W["dq"].T, eps) * W["dq.norm"]
    q = (cq @ W["uq"].T).view(T, H, D)
    c = rms(h @ W["dkv"].T, eps) * W["dkv.norm"]
    k = (c @ W["uk"].T).view(T, H, D)
    v = (c @ W["uv"].T).view(T, H, Dv)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~visible, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * Dv)
    return o @ W["o"].T


def dense_ff(h, W):
    return xielu(h @ W["up"].T, W["act"][0], W["act"][1]) @ W["down"].T


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, correction, r):
    """(chosen [T, top] indices, weights [T, top]) among experts + identity outputs"""
    n_out = router.shape[0]
    s = torch.softmax(h @ router.T, dim=-1)
    choice = s + correction
    groups = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = int(groups["count"]), int(groups["keep"])
    per = n_out // G
    best = choice.view(-1, G, per).max(-1).values                               # [T, G]
    kept = best.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
    allowed = allowed.repeat_interleave(per, dim=1)
    chosen = choice.masked_fill(~allowed, float("-inf")).topk(int(r["top"]), dim=-1).indices
    return chosen, s.gather(1, chosen)


def moe_ff(h, W, mlp):
    """W: the feed-forward's tensors by short name (router, correction, e<i>.gate/up/down, shared.gate/up/down)"""
    r = mlp["router"]
    E = int(r["experts"])
    chosen, weights = route(h, W["router"], W["correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            if e >= E:
                out[t] += w * h[t]
            else:
                out[t] += w * gated_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"])
    return out


def token_side(x, tokens, side_embed, layer, dim, W, eps):
    e = side_embed[torch.tensor(tokens, dtype=torch.int64)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W["gate"].T) * e) @ W["proj"].T
    return rms(y, eps) * W["norm"]


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg, w, tokens, collect=None):
    """logits [T, vocab] of one sequence.  ``collect``: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    emb = cfg["embedding"]
    bg = emb.get("bigram")
    x = embedding(tokens, w["embed"], emb["scale"], w.get("bigram") if bg else None, *( (bg["buckets"], bg["mul_prev"], bg["mul_cur"]) if bg else ()))
    streams = [x]
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = scalar_norm(latent_attention(x, sub(w, p + "mix."), lc["mixer"], eps), w[p + "norm1"], eps)
        x = x + (y * w[p + "ls1"] if p + "ls1" in w else y)
        if lc.get("mlp") is not None:
            W = sub(w, p + "mlp.")
            y = dense_ff(x, W) if lc["mlp"]["kind"] == "dense" else moe_ff(x, W, lc["mlp"])
            y = scalar_norm(y, w[p + "norm2"], eps)
            x = x + (y * w[p + "ls2"] if p + "ls2" in w else y)
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, w["side.embed"], i, cfg["token_side"]["dim"], sub(w, p + "side."), eps)
        streams.append(x)
        if p + "dwa" in w:
            x = sum(w[p + "dwa"][j] * streams[j] for j in range(i + 2))
        if collect is not None:
            collect.append(x)
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T


def windowed_attention(q, k, v, scale, window=0, first=0, held=0):
    """the general statement behind the attention kernel, by loops: q [S, H, D] are the queries of storage indices held .. held +
    S - 1; k [L, G, D], v [L, G, Dv] with H a multiple of G; index j is visible to the query at c when first <= j <= c and
    (window == 0 or c - j < window).  Queries in front of ``first`` give zeros."""
    S, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(S, H, v.shape[2], dtype=q.dtype)
    for t in range(S):
        c = held + t
        lo = max(first, c - window + 1 if window else 0, 0)
        if c < first:
            continue
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:c + 1, g] @ q[t, h]) * scale
            out[t, h] = torch.softmax(s, dim=0) @ v[lo:c + 1, g]
    return out


def greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens


# ------------------------------------------------------------------ random models for the tests
def random_config(width=48, vocab=61, heads=3, dim=8, vdim=12, q_rank=20, kv_rank=24, scale=0.3, ff=40, kinds=("dense", "moe", None),
                  experts=6, identity=3, groups=(3, 2), top=3, expert_ff=16, shared_ff=20, side_dim=5, bigram=(53, 31, 17), emb_scale=0.7,
                  eps=1e-5):
    """config.json of a small model; ``kinds``: per layer the feed-forward ("dense", "moe" or None)"""
    layers = []
    for kind in kinds:
        mlp = None
        if kind == "dense":
            mlp = {"kind": "dense", "ff": ff}
        elif kind == "moe":
            router = {"experts": experts, "identity": identity, "top": top}
            if groups is not None:
                router["groups"] = {"count": groups[0], "keep": groups[1]}
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": router}
            if shared_ff:
                mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": "latent_attention", "mlp": mlp,
                       "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}})
    cfg = {"architecture": "Serotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale}, "layers": layers}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if side_dim:
        cfg["token_side"] = {"dim": side_dim}
    return cfg


def random_weights(cfg, seed, layer_scale=True, depth_average=True):
    """checkpoint tensors (bfloat16, so that every dtype of the model starts from the same numbers)"""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def lin(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / math.sqrt(i)

    def near(n, centre, spread):
        return centre + spread * torch.randn(n, generator=g)

    w = {"embed": torch.randn(V, W, generator=g), "head": lin(V, W), "final.norm": near((), 1.0, 0.1)}
    bg = cfg["embedding"].get("bigram")
    if bg:
        w["bigram"] = torch.randn(bg["buckets"] + 1, W, generator=g) * 0.7
    side = cfg.get("token_side")
    if side:
        w["side.embed"] = torch.randn(V, side["dim"] * len(cfg["layers"]), generator=g)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        w[p + "mix.dq"], w[p + "mix.dq.norm"] = lin(m["q_rank"], W), near(m["q_rank"], 1.0, 0.2)
        w[p + "mix.uq"] = lin(H * D, m["q_rank"], 2.0)
        w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = lin(m["kv_rank"], W), near(m["kv_rank"], 1.0, 0.2)
        w[p + "mix.uk"], w[p + "mix.uv"] = lin(H * D, m["kv_rank"], 2.0), lin(H * Dv, m["kv_rank"])
        w[p + "mix.o"] = lin(W, H * Dv)
        w[p + "norm1"] = near((), 1.0, 0.1)
        if layer_scale:
            w[p + "ls1"] = near(W, 0.6, 0.15)
        mlp = lc["mlp"]
        if mlp is not None:
            w[p + "norm2"] = near((), 1.0, 0.1)
            if layer_scale:
                w[p + "ls2"] = near(W, 0.6, 0.15)
            if mlp["kind"] == "dense":
                w[p + "mlp.up"], w[p + "mlp.down"], w[p + "mlp.act"] = lin(mlp["ff"], W), lin(W, mlp["ff"]), torch.randn(2, generator=g)
            else:
                r = mlp["router"]
                n_out = r["experts"] + r.get("identity", 0)
                w[p + "mlp.router"], w[p + "mlp.correction"] = lin(n_out, W, 1.5), 0.05 * torch.randn(n_out, generator=g)
                names = [f"e{e}." for e in range(r["experts"])] + (["shared."] if mlp.get("shared") else [])
                for n in names:
                    f = mlp["shared"]["ff"] if n == "shared." else mlp["expert"]["ff"]
                    w[p + "mlp." + n + "gate"], w[p + "mlp." + n + "up"], w[p + "mlp." + n + "down"] = lin(f, W), lin(f, W), lin(W, f)
        if side:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = lin(side["dim"], W), lin(W, side["dim"]), near(W, 0.5, 0.1)
        if depth_average:
            c = torch.rand(i + 2, generator=g) + 0.2
            c[-1] += 1.0
            w[p + "dwa"] = c / c.sum() * near((), 1.0, 0.05)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}
