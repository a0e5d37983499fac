"""Slow, plain statements of the mechanisms of the Zafepel design, one function per mechanism, in whatever
floating-point type the inputs have (the tests use float64).  Test infrastructure only: nothing of the package is
imported here, and the package imports nothing from here.

Conventions shared by all functions: a batch row holds ``S`` new tokens that follow ``past`` tokens already seen;
row ``b`` of a batch is LEFT-padded by ``pad[b]`` tokens counted from the very first token the row ever saw, so the
token in slot ``c = past + t`` has position ``c - pad[b]`` and does not exist when that is negative.
"""
import math

import torch


# ------------------------------------------------------------------ element-wise pieces
def dyn_tanh(x, alpha, weight, bias):
    """Dynamic Tanh normalisation: tanh(alpha x) * weight + bias (no statistics of x)"""
    return torch.tanh(alpha * x) * weight + bias


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def poly_norm(z, coef, eps):
    """coef = (a, b, c, e):  a N(z) + b N(z^2) + c N(z^3) + e, N = rms_unit over the feature axis"""
    a, b, c, e = [coef[i] for i in range(4)]
    return a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e


def soft_cap(x, cap):
    return cap * torch.tanh(x / cap)


# ------------------------------------------------------------------ rotary, interleaved pairs, partial width
def rotate_pairs(x, positions, base, rot_dims):
    """x [..., n, D] with ``positions`` [...] broadcastable to x's leading axes (one per token).  Elements 2i and 2i+1
    (i < rot_dims / 2) turn by the angle position * base^(-2i/rot_dims); the rest of D passes."""
    out = x.clone()
    half = rot_dims // 2
    freq = torch.tensor([base ** (-2.0 * i / rot_dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[..., None, None] * freq                      # [..., 1, half]
    u, v = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
    out[..., 0:rot_dims:2] = u * torch.cos(ang) - v * torch.sin(ang)
    out[..., 1:rot_dims:2] = v * torch.cos(ang) + u * torch.sin(ang)
    return out


# ------------------------------------------------------------------ sigmoid attention over a sliding window
def sigmoid_window_attention(q, k_all, v_all, past, pad, window, scale, head_bias):
    """q [B, S, H, D] (new tokens, slots past .. past+S-1); k_all [B, L, G, D], v_all [B, L, G, Dv] hold every slot
    0 .. past+S-1.  Query slot c sees key slot j when 0 <= c - j < window and j is not padding.  The weight of a visible
    key is sigmoid(q.k * scale + head_bias[h]); weights are NOT normalised.  Returns [B, S, H, Dv]."""
    B, S, H, D = q.shape
    G, Dv = k_all.shape[2], v_all.shape[3]
    out = torch.zeros(B, S, H, Dv, dtype=q.dtype)
    for b in range(B):
        for t in range(S):
            c = past + t
            if c < pad[b]:
                continue
            lo = max(int(pad[b]), c - window + 1)
            for h in range(H):
                g = h // (H // G)
                s = (k_all[b, lo:c + 1, g] @ q[b, t, h]) * scale + head_bias[h]
                out[b, t, h] = torch.sigmoid(s) @ v_all[b, lo:c + 1, g]
    return out


# ------------------------------------------------------------------ short causal convolution per channel
def short_conv_silu(x, weight, tail, past, pad):
    """x [B, S, C]; weight [C, taps] (last column multiplies the current token); tail [B, taps-1, C] = the inputs of the
    taps-1 slots before this call (zeros at the start of a sequence).  Padding slots count as zeros.  Returns
    (silu(conv) [B, S, C], new tail)."""
    B, S, C = x.shape
    taps = weight.shape[1]
    x = x.clone()
    for b in range(B):
        n = max(0, int(pad[b]) - past)
        x[b, :n] = 0
    full = torch.cat([tail, x], dim=1)                                      # [B, taps-1+S, C]
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[:, j:j + S] * weight[:, j]
    return silu(y), full[:, S:].clone()


# ------------------------------------------------------------------ the two linear recurrences
def gated_delta_rule(q, k, v, beta, decay, state, past, pad):
    """q, k [B, S, G, D] (already unit vectors, q already scaled), v [B, S, H, Dv], beta and decay [B, S, H],
    state [B, H, D, Dv].  Per head and token:  M <- decay M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q.
    Returns (o [B, S, H, Dv], new state)."""
    B, S, H, Dv = v.shape
    G = q.shape[2]
    state = state.clone()
    o = torch.zeros(B, S, H, Dv, dtype=v.dtype)
    for b in range(B):
        for t in range(S):
            if past + t < pad[b]:
                continue
            for h in range(H):
                g = h // (H // G)
                M = state[b, h] * decay[b, t, h]
                u = beta[b, t, h] * (v[b, t, h] - M.t() @ k[b, t, g])
                M = M + torch.outer(k[b, t, g], u)
                state[b, h] = M
                o[b, t, h] = M.t() @ q[b, t, g]
    return o, state


def gated_linear_attention(q, k, v, alpha, state, past, pad):
    """q, k, alpha [B, S, H, D], v [B, S, H, Dv], state [B, H, D, Dv]:  M <- diag(alpha) M + k v^T;  o = M^T q."""
    B, S, H, Dv = v.shape
    state = state.clone()
    o = torch.zeros(B, S, H, Dv, dtype=v.dtype)
    for b in range(B):
        for t in range(S):
            if past + t < pad[b]:
                continue
            for h in range(H):
                M = alpha[b, t, h][:, None] * state[b, h] + torch.outer(k[b, t, h], v[b, t, h])
                state[b, h] = M
                o[b, t, h] = M.t() @ q[b, t, h]
    return o, state


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


# ------------------------------------------------------------------ a whole model, from a dict of parameters
class OracleModel:
    """``cfg`` is the dict of config.json, ``w`` maps the checkpoint's tensor names to tensors (any float type; they are
    converted to ``dtype``).  ``forward`` runs S new tokens of a left-padded batch and keeps every slot of every layer
    run (no window eviction, no pages): the slowest correct statement."""

    def __init__(self, cfg, w, dtype=torch.float64):
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: v.to(dtype) for k, v in w.items()}
        lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 0}
        n = len(cfg["layers"])
        self.runs, self.pass_start = [], {}
        self.runs += list(range(0, lp["start"]))
        for t in range(lp["times"]):
            self.pass_start[len(self.runs)] = t
            self.runs += list(range(lp["start"], lp["stop"]))
        self.runs += list(range(lp["stop"] if lp["times"] else lp["start"], n))
        self.eps = cfg["norm"]["eps"]

    def new_state(self):
        return {"past": 0, "pad": None, "runs": [dict() for _ in self.runs]}

    def _norm(self, name, x):
        return dyn_tanh(x, self.w[name + ".alpha"], self.w[name], self.w[name + ".b"])

    def _lin(self, name, x, bias=False):
        y = x @ self.w[name].t()
        return y + self.w[name + ".b"] if bias else y

    def _left(self, p, m, h, st, past, pad):
        B, S, _ = h.shape
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q = self._lin(p + "q", h, True).view(B, S, H, D)
        k = self._lin(p + "k", h, True).view(B, S, G, D)
        v = self._lin(p + "v", h, True).view(B, S, G, Dv)
        q = rms_unit(q, self.eps) * self.w[p + "q.norm"]
        k = rms_unit(k, self.eps) * self.w[p + "k.norm"]
        pos = (past + torch.arange(S))[None, :] - pad[:, None]                 # [B, S]
        q = rotate_pairs(q, pos, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_pairs(k, pos, m["rot"]["base"], m["rot"]["dims"])
        st["k"] = torch.cat([st["k"], k], 1) if "k" in st else k
        st["v"] = torch.cat([st["v"], v], 1) if "v" in st else v
        o = sigmoid_window_attention(q, st["k"], st["v"], past, pad, m["mask"]["size"], m["scale"], self.w[p + "pb"])
        return self._lin(p + "o", o.reshape(B, S, H * Dv))

    def _right(self, p, m, h, st, past, pad):
        B, S, _ = h.shape
        H, G, D, Dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        outs = []
        for name, width in (("q", G * D), ("k", G * D), ("v", H * Dv)):
            tail = st.get("tail_" + name, torch.zeros(B, taps - 1, width, dtype=self.dtype))
            y, st["tail_" + name] = short_conv_silu(self._lin(p + name, h), self.w[p + name + ".conv"], tail, past, pad)
            outs.append(y)
        q = unit_vector(outs[0].view(B, S, G, D)) * D ** -0.5
        k = unit_vector(outs[1].view(B, S, G, D))
        v = outs[2].view(B, S, H, Dv)
        beta = torch.sigmoid(self._lin(p + "b", h))
        decay = torch.exp(-torch.exp(self.w[p + "A_log"]) * torch.nn.functional.softplus(self._lin(p + "a", h) + self.w[p + "dt_bias"]))
        state = st.get("M", torch.zeros(B, H, D, Dv, dtype=self.dtype))
        o, st["M"] = gated_delta_rule(q, k, v, beta, decay, state, past, pad)
        o = rms_unit(o, self.eps) * self.w[p + "norm"] * silu(self._lin(p + "g", h)).view(B, S, H, Dv)
        return self._lin(p + "o", o.reshape(B, S, H * Dv))

    def _gla(self, p, m, h, st, past, pad):
        B, S, _ = h.shape
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        q = (self._lin(p + "q", h) * D ** -0.5).view(B, S, H, D)
        k = self._lin(p + "k", h).view(B, S, H, D)
        v = self._lin(p + "v", h).view(B, S, H, Dv)
        z = self._lin(p + "a2", self._lin(p + "a1", h), True)
        alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(B, S, H, D)
        state = st.get("M", torch.zeros(B, H, D, Dv, dtype=self.dtype))
        o, st["M"] = gated_linear_attention(q, k, v, alpha, state, past, pad)
        o = (rms_unit(o, self.eps) * self.w[p + "norm"]).reshape(B, S, H * Dv) * silu(self._lin(p + "g", h))
        return self._lin(p + "o", o)

    def forward(self, ids, state, pad=None, collect=None):
        """ids [B, S] (left-padded on a sequence's first call); returns logits [B, S, vocab]"""
        B, S = ids.shape
        if state["pad"] is None:
            state["pad"] = torch.zeros(B, dtype=torch.long) if pad is None else pad.clone()
        pad, past = state["pad"], state["past"]
        x = self.w["embed"][ids]
        for r, li in enumerate(self.runs):
            if r in self.pass_start:
                x = x + self.w["loop.step"][self.pass_start[r]]
            lc, p, st = self.cfg["layers"][li], "l%d." % li, state["runs"][r]
            h = self._norm(p + "norm1", x)
            if lc["type"] == "parallel":
                m = lc["mixer"]
                y = m["left_scale"] * self._left(p + "mix.left.", m["left"], h, st.setdefault("L", {}), past, pad) \
                    + m["right_scale"] * self._right(p + "mix.right.", m["right"], h, st.setdefault("R", {}), past, pad)
            else:
                y = self._gla(p + "mix.", lc["mixer"], h, st, past, pad)
            x = x + self._norm(p + "norm1b", y)
            if lc.get("mlp") is not None:
                z = self._lin(p + "mlp.up", self._norm(p + "norm2", x))
                x = x + self._norm(p + "norm2b", self._lin(p + "mlp.down", poly_norm(z, self.w[p + "mlp.act"], self.eps)))
            if collect is not None:
                collect.append(x.clone())
        state["past"] = past + S
        logits = self._lin("head", self._norm("final.norm", x))
        cap = self.cfg.get("logit_softcap")
        return soft_cap(logits, cap) if cap else logits


# ------------------------------------------------------------------ random small models for the tests
def random_config(seed, width=64, vocab=97, order=("parallel", "gla", "parallel"), loop=(1, 2, 2), window=5, heads=4, kv_heads=2,
                  dim=12, vdim=10, rot_dims=8, r_heads=4, r_kv_heads=2, r_dim=6, r_vdim=9, taps=4, g_heads=3, g_dim=7, g_vdim=5,
                  rank=5, ff=40, tau=8.0, mlp_on=(True, False, True), softcap=20.0, eps=1e-5):
    layers = []
    for i, kind in enumerate(order):
        if kind == "parallel":
            mixer = {"left": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
                              "rot": {"base": 100.0 + 7 * i, "dims": rot_dims}, "scale": 1.7 / math.sqrt(dim), "vdim": vdim},
                     "left_scale": 0.7, "right": {"conv": taps, "dim": r_dim, "heads": r_heads, "kv_heads": r_kv_heads, "vdim": r_vdim},
                     "right_scale": 1.2}
        else:
            mixer = {"dim": g_dim, "heads": g_heads, "tau": tau, "vdim": g_vdim, "rank": rank}
        layers.append({"type": kind, "mixer": mixer, "mlp": {"ff": ff, "kind": "dense"} if mlp_on[i % len(mlp_on)] else None})
    cfg = {"architecture": "Zafepel", "layers": layers, "logit_softcap": softcap, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed, dtype=torch.bfloat16):
    """checkpoint-named tensors; magnitudes chosen so that every branch matters (attention weights away from 0 and 1,
    decays between 0.5 and 1, recurrent states of order 1)"""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    w = {}

    def mat(name, o, i, s=1.0):
        w[name] = torch.randn(o, i, generator=g) * s / math.sqrt(i)

    def vec(name, n, mean=0.0, s=1.0):
        w[name] = mean + s * torch.randn(n, generator=g)

    def norm(name, n=W):
        vec(name, n, 1.0, 0.1)
        vec(name + ".b", n, 0.0, 0.1)
        w[name + ".alpha"] = torch.tensor(0.6) + 0.2 * torch.rand((), generator=g)

    w["embed"] = torch.randn(cfg["vocab"], W, generator=g)
    lp = cfg.get("loop")
    if lp:
        vec("loop.step", lp["times"] * W, 0.0, 0.5)
        w["loop.step"] = w["loop.step"].view(lp["times"], W)
    for i, lc in enumerate(cfg["layers"]):
        p = "l%d." % i
        norm(p + "norm1"); norm(p + "norm1b")
        if lc["mlp"] is not None:
            norm(p + "norm2"); norm(p + "norm2b")
            mat(p + "mlp.up", lc["mlp"]["ff"], W); mat(p + "mlp.down", W, lc["mlp"]["ff"])
            w[p + "mlp.act"] = torch.tensor([0.8, 0.5, -0.3, 0.1]) + 0.1 * torch.randn(4, generator=g)
        m = lc["mixer"]
        if lc["type"] == "parallel":
            l, r = m["left"], m["right"]
            q = p + "mix.left."
            mat(q + "q", l["heads"] * l["dim"], W); vec(q + "q.b", l["heads"] * l["dim"], 0, 0.2)
            mat(q + "k", l["kv_heads"] * l["dim"], W); vec(q + "k.b", l["kv_heads"] * l["dim"], 0, 0.2)
            mat(q + "v", l["kv_heads"] * l["vdim"], W); vec(q + "v.b", l["kv_heads"] * l["vdim"], 0, 0.2)
            vec(q + "q.norm", l["dim"], 1.0, 0.2); vec(q + "k.norm", l["dim"], 1.0, 0.2)
            vec(q + "pb", l["heads"], -1.0, 0.5)
            mat(q + "o", W, l["heads"] * l["vdim"])
            q = p + "mix.right."
            for n_, c in (("q", r["kv_heads"] * r["dim"]), ("k", r["kv_heads"] * r["dim"]), ("v", r["heads"] * r["vdim"])):
                mat(q + n_, c, W, 2.0)
                w[q + n_ + ".conv"] = torch.randn(c, r["conv"], generator=g) * 0.6
            mat(q + "b", r["heads"], W); mat(q + "a", r["heads"], W)
            vec(q + "A_log", r["heads"], -1.0, 0.5); vec(q + "dt_bias", r["heads"], 0.0, 0.5)
            vec(q + "norm", r["vdim"], 1.0, 0.2)
            mat(q + "g", r["heads"] * r["vdim"], W); mat(q + "o", W, r["heads"] * r["vdim"])
        else:
            q = p + "mix."
            rank = m.get("rank", 4)
            mat(q + "q", m["heads"] * m["dim"], W); mat(q + "k", m["heads"] * m["dim"], W); mat(q + "v", m["heads"] * m["vdim"], W)
            mat(q + "g", m["heads"] * m["vdim"], W); mat(q + "o", W, m["heads"] * m["vdim"])
            vec(q + "norm", m["vdim"], 1.0, 0.2)
            mat(q + "a1", rank, W); mat(q + "a2", m["heads"] * m["dim"], rank, 2.0); vec(q + "a2.b", m["heads"] * m["dim"], 2.0, 1.0)
    norm("final.norm")
    mat("head", cfg["vocab"], W, 2.0)
    out = {k: v.to(dtype) for k, v in w.items()}
    for lc in cfg["layers"]:
        lc["mixer"].pop("rank", None)
    return out
