"""Zafepel: a decoder-only design whose layers mix sequence positions in one of two ways,

* ``parallel``: a sliding-window attention with sigmoid weights (no softmax, a bias per head) next to a gated delta-rule
  recurrence behind short causal convolutions, both reading the same normalised input, their outputs summed with fixed scales;
* ``gla``: gated linear attention, a matrix state per head that decays per key channel;

with Dynamic-Tanh normalisation before and after every sublayer, a PolyNorm feed-forward on some layers, a block of layers
that runs several times with the same weights (each pass with its own state and an additive per-pass vector), and a
soft-capped output.  No library ships this model: the module tree, the configuration reader and the checkpoint's name map live
here, the state in ``transformers/kv.py`` (``DynamicStateCache``), the kernels in ``csrc/mixers`` behind
``ggml/model/mixers_cpp.py``.  The projections are ``nn.Linear`` modules (merged per mixer by ``merge_projections``), so the
low-bit conversion treats them like any other model's; the residual stream, every normalisation, the attention scores and
everything inside the recurrences are 32-bit whatever the model's dtype.
"""
import json
import math
import os
from typing import Optional

import torch
from torch import nn
from transformers import GenerationMixin, PreTrainedConfig, PreTrainedModel
from transformers.modeling_outputs import CausalLMOutputWithPast

from ipex_llm_b200.transformers.kv import DynamicStateCache
from ipex_llm_b200.transformers.models import mixer_ops as ops
from ipex_llm_b200.transformers.models.common import merge_linear, merge_linear_inputs
from ipex_llm_b200.transformers.models.utils import read_safetensors
from ipex_llm_b200.utils.common import invalidInputError


class ZafepelConfig(PreTrainedConfig):
    """config.json of the design: ``vocab``, ``width``, ``layers`` (per layer: ``type``, ``mixer`` sizes, ``mlp`` or null),
    ``loop`` (``start``, ``stop``, ``times``; optional), ``norm.eps``, ``logit_softcap`` (optional)."""
    model_type = "zafepel"

    def __init__(self, vocab=256, width=64, layers=None, loop=None, norm=None, logit_softcap=None, architecture="Zafepel",
                 gla_ranks=None, **kwargs):
        self.vocab, self.width = int(vocab), int(width)
        # the rank of each gla layer's decay projection: not a key of the design's config.json (the loader reads it off the
        # checkpoint's shapes); kept here so that a saved model can be rebuilt from its configuration alone
        self.gla_ranks = {str(k): int(v) for k, v in (gla_ranks or {}).items()}
        self.layers = layers or []
        self.loop = loop
        self.norm = norm or {"eps": 1e-6}
        self.logit_softcap = logit_softcap
        self.architecture = architecture
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)
        # the names the rest of the framework reads
        self.vocab_size, self.hidden_size, self.num_hidden_layers = self.vocab, self.width, len(self.layers)
        self.use_cache = True

    @property
    def norm_eps(self):
        return float(self.norm["eps"])

    def layer_runs(self):
        """[(layer index, pass number or None)]: the order in which the layers run; a pass number marks the first layer of a
        pass of the repeated block (the pass vector is added right before it)"""
        n = len(self.layers)
        lp = self.loop
        if not lp or int(lp.get("times", 0)) < 1 or lp["stop"] <= lp["start"]:
            return [(i, None) for i in range(n)]
        runs = [(i, None) for i in range(0, lp["start"])]
        for t in range(int(lp["times"])):
            runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
        return runs + [(i, None) for i in range(lp["stop"], n)]


class DynamicTanh(nn.Module):
    """y = tanh(alpha x) * weight + bias"""

    def __init__(self, width):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width))
        self.bias = nn.Parameter(torch.zeros(width))
        self.alpha = nn.Parameter(torch.ones(()))


class _Weight(nn.Module):
    """a lone vector (a per-head RMS weight) under the name ``<module>.weight``"""

    def __init__(self, n):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))


class SigmoidWindowAttention(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        invalidInputError(self.heads % self.kv_heads == 0, "heads must be a multiple of kv_heads")
        self.window, self.scale = int(m["mask"]["size"]), float(m["scale"])
        self.rot_dims, self.rot_base = int(m["rot"]["dims"]), float(m["rot"]["base"])
        invalidInputError(self.rot_dims % 2 == 0 and self.rot_dims <= self.dim, "rot.dims must be even and at most dim")
        self.q_proj = nn.Linear(width, self.heads * self.dim, bias=True)
        self.k_proj = nn.Linear(width, self.kv_heads * self.dim, bias=True)
        self.v_proj = nn.Linear(width, self.kv_heads * self.vdim, bias=True)
        self.q_norm, self.k_norm = _Weight(self.dim), _Weight(self.dim)
        self.pos_bias = nn.Parameter(torch.zeros(self.heads))
        self.o_proj = nn.Linear(self.heads * self.vdim, width, bias=False)
        self._inv_freq = {}

    def inv_freq(self, device):
        """base^(-2i/rot_dims), i < rot_dims / 2, in double precision (the kernel forms the angles in double precision too).
        Not a buffer: ``model.to(dtype)`` must not round it."""
        t = self._inv_freq.get(device)
        if t is None:
            freq = [self.rot_base ** (-2.0 * i / self.rot_dims) for i in range(self.rot_dims // 2)] or [0.0]    # never empty
            t = self._inv_freq[device] = torch.tensor(freq, dtype=torch.float64).to(device)
        return t

    def out_width(self):
        return self.heads * self.vdim


class GatedDeltaRule(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], int(m["conv"])
        invalidInputError(self.heads % self.kv_heads == 0, "heads must be a multiple of kv_heads")
        qk, v = self.kv_heads * self.dim, self.heads * self.vdim
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(width, qk, bias=False), nn.Linear(width, qk, bias=False), nn.Linear(width, v, bias=False)
        self.conv_weight = nn.Parameter(torch.zeros(2 * qk + v, self.taps))     # rows in the order q, k, v
        self.b_proj, self.a_proj = nn.Linear(width, self.heads, bias=False), nn.Linear(width, self.heads, bias=False)
        self.A_log, self.dt_bias = nn.Parameter(torch.zeros(self.heads)), nn.Parameter(torch.zeros(self.heads))
        self.norm = _Weight(self.vdim)
        self.g_proj = nn.Linear(width, v, bias=False)
        self.o_proj = nn.Linear(v, width, bias=False)

    def out_width(self):
        return self.heads * self.vdim


class ParallelMixer(nn.Module):
    """attention (``left``) and delta rule (``right``) on the same input; ``in_proj`` / ``out_proj`` appear when
    ``merge_projections`` has run: one matrix product in, one out (the sum of the two branches happens in its accumulator)"""

    def __init__(self, width, m):
        super().__init__()
        self.left, self.right = SigmoidWindowAttention(width, m["left"]), GatedDeltaRule(width, m["right"])
        self.left_scale, self.right_scale = float(m["left_scale"]), float(m["right_scale"])


class GatedLinearAttention(nn.Module):
    def __init__(self, width, m, rank):
        super().__init__()
        self.heads, self.dim, self.vdim, self.tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
        qk, v = self.heads * self.dim, self.heads * self.vdim
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(width, qk, bias=False), nn.Linear(width, qk, bias=False), nn.Linear(width, v, bias=False)
        self.g_proj = nn.Linear(width, v, bias=False)
        self.a1_proj, self.a2_proj = nn.Linear(width, rank, bias=False), nn.Linear(rank, qk, bias=True)
        self.norm = _Weight(self.vdim)
        self.o_proj = nn.Linear(v, width, bias=False)


class PolyNormMLP(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        invalidInputError(m.get("kind", "dense") == "dense", f"unknown feed-forward kind {m.get('kind')}")
        self.up_proj, self.down_proj = nn.Linear(width, m["ff"], bias=False), nn.Linear(m["ff"], width, bias=False)
        self.act = nn.Parameter(torch.zeros(4))


class ZafepelLayer(nn.Module):
    def __init__(self, width, lc, rank):
        super().__init__()
        self.kind = lc["type"]
        invalidInputError(self.kind in ("parallel", "gla"), f"unknown layer type {self.kind}")
        self.norm1, self.norm1b = DynamicTanh(width), DynamicTanh(width)
        self.mixer = ParallelMixer(width, lc["mixer"]) if self.kind == "parallel" else GatedLinearAttention(width, lc["mixer"], rank)
        self.mlp = None
        if lc.get("mlp") is not None:
            self.norm2, self.norm2b = DynamicTanh(width), DynamicTanh(width)
            self.mlp = PolyNormMLP(width, lc["mlp"])


def _zero_rows(like: nn.Linear, rows_so_far: int, multiple: int):
    """a bias-free projection of zeros that brings a merged row count up to a multiple (none when it is one already)"""
    extra = -rows_so_far % multiple if multiple else 0
    if not extra:
        return []
    with torch.device("meta"):
        pad = nn.Linear(1, 1, bias=False)
    pad.weight = nn.Parameter(torch.zeros(extra, like.weight.shape[1], dtype=like.weight.dtype, device=like.weight.device), requires_grad=False)
    return [pad]


def merge_projections(module: nn.Module, row_multiple: int = 0):
    """every projection that reads the mixer's input becomes one ``in_proj``; the two output projections of a parallel mixer
    become one ``out_proj`` over the concatenated branch outputs.  ``row_multiple``: rows of zeros are appended to ``in_proj`` up
    to a multiple of it (the low-bit prefill GEMM wants whole 128-row tiles; the few gate / rank rows would otherwise push the
    whole projection onto the general path); the kernels address columns by offset, the extra ones are never read."""
    if isinstance(module, ParallelMixer) and not hasattr(module, "in_proj"):
        l, r = module.left, module.right
        parts = [l.q_proj, l.k_proj, l.v_proj, r.q_proj, r.k_proj, r.v_proj, r.b_proj, r.a_proj, r.g_proj]
        module.in_proj = merge_linear(parts + _zero_rows(l.q_proj, sum(p.weight.shape[0] for p in parts), row_multiple))
        module.out_proj = merge_linear_inputs([l.o_proj, r.o_proj])
        del l.q_proj, l.k_proj, l.v_proj, l.o_proj, r.q_proj, r.k_proj, r.v_proj, r.b_proj, r.a_proj, r.g_proj, r.o_proj
    elif isinstance(module, GatedLinearAttention) and not hasattr(module, "in_proj"):
        parts = [module.q_proj, module.k_proj, module.v_proj, module.g_proj, module.a1_proj]
        module.in_proj = merge_linear(parts + _zero_rows(module.q_proj, sum(p.weight.shape[0] for p in parts), row_multiple))
        del module.q_proj, module.k_proj, module.v_proj, module.g_proj, module.a1_proj


class ZafepelModel(nn.Module):
    def __init__(self, config: ZafepelConfig, ranks):
        super().__init__()
        self.config = config
        w = config.width
        self.embed_tokens = nn.Embedding(config.vocab, w)
        times = int(config.loop["times"]) if config.loop else 0
        self.loop_step = nn.Parameter(torch.zeros(max(times, 1), w)) if times else None
        self.layers = nn.ModuleList([ZafepelLayer(w, lc, ranks.get(i, 1)) for i, lc in enumerate(config.layers)])
        self.norm = DynamicTanh(w)


def _lin(linear, x):
    """a projection on [N, in] rows: cuBLAS for nn.Linear, the low-bit kernels for a converted module"""
    return linear(x)


class ZafepelForCausalLM(PreTrainedModel, GenerationMixin):
    config_class = ZafepelConfig
    base_model_prefix = "model"
    _no_split_modules = ["ZafepelLayer"]
    _supports_attention_backend = False
    main_input_name = "input_ids"

    def __init__(self, config: ZafepelConfig, ranks=None):
        super().__init__(config)
        if ranks is None:
            ranks = {int(k): v for k, v in config.gla_ranks.items()}
        config.gla_ranks = {str(k): int(v) for k, v in ranks.items()}
        self.model = ZafepelModel(config, ranks)
        self.lm_head = nn.Linear(config.width, config.vocab, bias=False)
        self.collect_residual = None          # a list: gets the residual stream after every layer run (debugging aid)

    def _init_weights(self, module):
        pass

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    # ---- the mixers (x: fp32 residual [N, W]; h: the normalised input, model dtype, [N, W])
    def _parallel(self, mx, h, st, B, S, cache):
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        l, r = mx.left, mx.right
        proj = _lin(mx.in_proj, h)                                           # [N, P]
        P = proj.shape[1]
        proj = proj.view(B, S, P)
        eps = self.config.norm_eps
        out = torch.empty(B * S, l.out_width() + r.out_width(), dtype=h.dtype, device=h.device)
        # left: q | k | v  -> per-head RMS norm, rotary, cache append; then the windowed sigmoid attention
        off_k = l.heads * l.dim
        off_v = off_k + l.kv_heads * l.dim
        off_r = off_v + l.kv_heads * l.vdim
        kv = st.kv
        like_k = torch.empty((B, l.kv_heads, 0, l.dim), dtype=h.dtype, device=h.device)
        like_v = torch.empty((B, l.kv_heads, 0, l.vdim), dtype=h.dtype, device=h.device)
        k_store, v_store, held = kv.slots(like_k, like_v, S)
        shift = cache.seen - held                                            # storage index + shift = slot number
        # a recorded decode step reads the length from the device (the value given here is the one at recording time)
        dyn = kv.length_dev if (cache.frozen and S == 1) else None
        q = ops.window_qk_prepare(proj, 0, off_k, off_v, l.heads, l.kv_heads, l.dim, l.vdim, l.q_norm.weight, l.k_norm.weight,
                                  eps, l.inv_freq(h.device), l.rot_dims, k_store, v_store, kv.capacity(), held, shift, cache.pad, dyn)
        kv.commit(S)
        ops.sigmoid_window_attention(q, k_store, v_store, kv.capacity(), held, shift, cache.pad, l.window, l.scale, l.pos_bias,
                                     out, 0, mx.left_scale, dyn)
        # right: q | k | v (convolved) | beta | decay | gate
        qk = r.kv_heads * r.dim
        C = 2 * qk + r.heads * r.vdim
        off_b = off_r + C
        off_a = off_b + r.heads
        off_g = off_a + r.heads
        tail, tail_next = st.rec.tails(B, r.taps, C, h.dtype, h.device)
        pad = cache.pad if cache.seen == 0 else None                         # padding only ever precedes a row's first call
        if S == 1:                                                           # one thread per channel: the tail is shifted in place
            conv = ops.short_conv_silu(proj, off_r, C, r.conv_weight, tail, tail, cache.seen, pad)
        else:
            conv = ops.short_conv_silu(proj, off_r, C, r.conv_weight, tail, tail_next, cache.seen, pad)
            tail.copy_(tail_next)                                            # the tail keeps its address (a recorded step holds it)
        state = st.rec.matrix(B, r.heads, r.dim, r.vdim, h.device)
        o = ops.gated_delta_rule(conv, r.kv_heads, r.heads, r.dim, r.vdim, proj, off_b, off_a, r.A_log, r.dt_bias, state,
                                 cache.seen, pad)
        ops.gated_rms_norm(o, proj, off_g, r.norm.weight, eps, out, l.out_width(), mx.right_scale)
        return _lin(mx.out_proj, out)

    def _gla(self, mx, h, st, B, S, cache):
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        proj = _lin(mx.in_proj, h)
        P = proj.shape[1]
        qk, v = mx.heads * mx.dim, mx.heads * mx.vdim
        off_g = 2 * qk + v
        off_a1 = off_g + v
        z = _lin(mx.a2_proj, proj[:, off_a1:off_a1 + mx.a2_proj.in_features])  # [N, H * D] decay logits
        state = st.rec.matrix(B, mx.heads, mx.dim, mx.vdim, h.device)
        o = ops.gated_linear_attention(proj.view(B, S, P), mx.heads, mx.dim, mx.vdim, z.view(B, S, qk), mx.tau, state,
                                       cache.seen, cache.pad if cache.seen == 0 else None)
        out = torch.empty(B * S, v, dtype=h.dtype, device=h.device)
        ops.gated_rms_norm(o, proj.view(B, S, P), off_g, mx.norm.weight, self.config.norm_eps, out, 0, 1.0)
        return _lin(mx.o_proj, out)

    def forward(self, input_ids: Optional[torch.LongTensor] = None, attention_mask: Optional[torch.Tensor] = None,
                position_ids=None, past_key_values=None, inputs_embeds=None, use_cache: Optional[bool] = None,
                logits_to_keep=0, **kwargs):
        """``input_ids`` [B, S]: the next S tokens of every row.  On the first call of a batch ``attention_mask`` [B, S] gives
        the left padding; later calls continue from ``past_key_values`` (a ``DynamicStateCache``; any other or no cache
        starts a new one).  Positions follow from the padding, ``position_ids`` is not read.  ``logits_to_keep``: 0 = all
        positions, n = the last n, or a 1-D tensor of positions."""
        invalidInputError(input_ids is not None and inputs_embeds is None, "the model takes token ids")
        core, cfg = self.model, self.config
        B, S = input_ids.shape
        dev, dtype = core.embed_tokens.weight.device, core.embed_tokens.weight.dtype
        cache = past_key_values
        if not isinstance(cache, DynamicStateCache):
            invalidInputError(cache is None or cache.get_seq_length() == 0, "a filled cache of another class cannot be continued")
            cache = DynamicStateCache()
        if cache.seen == 0:                                                  # a batch's first call: the mask gives the padding
            cache.start(attention_mask, B, S, dev)
        invalidInputError(cache.pad.shape[0] == B, "batch size differs from the cache's")
        x = ops.embed_rows(core.embed_tokens.weight, input_ids.reshape(-1))  # fp32 [N, W]
        pending = None                                                       # (sublayer output, its post-norm) not yet added to x
        for run, (li, loop_pass) in enumerate(cfg.layer_runs()):
            layer = core.layers[li]
            add = core.loop_step[loop_pass] if loop_pass is not None else None
            h = ops.dyt_residual_norm(x, pending, add, layer.norm1, dtype)
            if layer.kind == "parallel":
                st = cache.run_state(run, layer.mixer.left.window)
                y = self._parallel(layer.mixer, h, st, B, S, cache)
            else:
                st = cache.run_state(run)
                y = self._gla(layer.mixer, h, st, B, S, cache)
            pending = (y, layer.norm1b)
            if layer.mlp is not None:
                h = ops.dyt_residual_norm(x, pending, None, layer.norm2, dtype)
                z = _lin(layer.mlp.up_proj, h)
                y = _lin(layer.mlp.down_proj, ops.poly_norm(z, layer.mlp.act, cfg.norm_eps))
                pending = (y, layer.norm2b)
            if self.collect_residual is not None:
                ops.dyt_residual_norm(x, pending, None, None, dtype)
                pending = None
                self.collect_residual.append(x.view(B, S, -1).clone())
        cache.advance(S)
        if isinstance(logits_to_keep, int) and logits_to_keep == 0:
            h = ops.dyt_residual_norm(x, pending, None, core.norm, dtype).view(B, S, -1)
        else:
            ops.dyt_residual_norm(x, pending, None, None, dtype)
            idx = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep.to(dev)
            xk = x.view(B, S, -1)[:, idx, :].contiguous()
            h = ops.dyt_residual_norm(xk.view(-1, xk.shape[-1]), None, None, core.norm, dtype).view(B, xk.shape[1], -1)
        # every kept position as a row of its own ([rows, 1, W]): a converted lm_head keeps only the last position of a long
        # sequence axis (the reference's prefill shortcut), and which positions to keep is decided here, by logits_to_keep
        logits = _lin(self.lm_head, h.reshape(-1, 1, h.shape[-1]))
        logits = ops.soft_cap(logits, cfg.logit_softcap).view(B, h.shape[1], -1)          # fp32
        return CausalLMOutputWithPast(logits=logits, past_key_values=cache)

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kwargs):
        """generate() hands over every token so far; the model takes those its cache has not seen"""
        seen = past_key_values.get_seq_length() if isinstance(past_key_values, DynamicStateCache) else 0
        return {"input_ids": input_ids[:, seen:], "attention_mask": attention_mask, "past_key_values": past_key_values,
                "use_cache": True, "logits_to_keep": 1}


# ------------------------------------------------------------------ checkpoint
def checkpoint_key_map(config: ZafepelConfig):
    """the model's parameter names -> the checkpoint's tensor names (or a list of them, concatenated by rows)"""
    m = {"model.embed_tokens.weight": "embed", "lm_head.weight": "head"}
    if config.loop and int(config.loop.get("times", 0)):
        m["model.loop_step"] = "loop.step"

    def norm(dst, src):
        m[dst + ".weight"], m[dst + ".bias"], m[dst + ".alpha"] = src, src + ".b", src + ".alpha"

    norm("model.norm", "final.norm")
    for i, lc in enumerate(config.layers):
        d, s = f"model.layers.{i}.", f"l{i}."
        norm(d + "norm1", s + "norm1")
        norm(d + "norm1b", s + "norm1b")
        if lc.get("mlp") is not None:
            norm(d + "norm2", s + "norm2")
            norm(d + "norm2b", s + "norm2b")
            m[d + "mlp.up_proj.weight"], m[d + "mlp.down_proj.weight"], m[d + "mlp.act"] = s + "mlp.up", s + "mlp.down", s + "mlp.act"
        if lc["type"] == "parallel":
            dl, sl = d + "mixer.left.", s + "mix.left."
            for n in ("q", "k", "v"):
                m[dl + n + "_proj.weight"], m[dl + n + "_proj.bias"] = sl + n, sl + n + ".b"
            m[dl + "q_norm.weight"], m[dl + "k_norm.weight"] = sl + "q.norm", sl + "k.norm"
            m[dl + "pos_bias"], m[dl + "o_proj.weight"] = sl + "pb", sl + "o"
            dr, sr = d + "mixer.right.", s + "mix.right."
            for n in ("q", "k", "v", "b", "a", "g", "o"):
                m[dr + n + "_proj.weight"] = sr + n
            m[dr + "conv_weight"] = [sr + "q.conv", sr + "k.conv", sr + "v.conv"]
            m[dr + "A_log"], m[dr + "dt_bias"], m[dr + "norm.weight"] = sr + "A_log", sr + "dt_bias", sr + "norm"
        else:
            dm, sm = d + "mixer.", s + "mix."
            for n in ("q", "k", "v", "g", "o", "a1", "a2"):
                m[dm + n + "_proj.weight"] = sm + n
            m[dm + "a2_proj.bias"], m[dm + "norm.weight"] = sm + "a2.b", sm + "norm"
    return m


def load_pretrained(model_dir, torch_dtype=None, device=None):
    """config.json + model.safetensors of the design -> a ``ZafepelForCausalLM`` with its projections merged.  Sizes that
    config.json does not state (the rank of the decay projection) come from the tensors' shapes."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    config = ZafepelConfig(**raw)
    tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    ranks = {i: tensors[f"l{i}.mix.a1"].shape[0] for i, lc in enumerate(config.layers) if lc["type"] == "gla"}
    if torch_dtype in (None, "auto"):
        torch_dtype = tensors["embed"].dtype
    with torch.device("meta"):
        model = ZafepelForCausalLM(config, ranks)
    state = {}
    for dst, src in checkpoint_key_map(config).items():
        missing = [s for s in ([src] if isinstance(src, str) else src) if s not in tensors]
        invalidInputError(not missing, f"the checkpoint has no tensor {missing}")
        t = tensors[src] if isinstance(src, str) else torch.cat([tensors[s] for s in src], dim=0)
        state[dst] = t.to(torch_dtype)
    expected = dict(model.named_parameters())
    for name, p in expected.items():
        invalidInputError(name in state, f"no checkpoint tensor for parameter {name}")
        invalidInputError(tuple(state[name].shape) == tuple(p.shape),
                          f"{name}: checkpoint shape {tuple(state[name].shape)} but the configuration gives {tuple(p.shape)}")
    model.load_state_dict(state, strict=True, assign=True)
    model.eval()
    model.requires_grad_(False)
    model.config.dtype = torch_dtype
    if device is not None:
        model = model.to(device)
    return model


# the loaders that go through transformers' Auto classes (load_low_bit builds the architecture from a saved configuration)
def _register():
    from transformers import AutoConfig, AutoModelForCausalLM
    try:
        AutoConfig.register("zafepel", ZafepelConfig)
        AutoModelForCausalLM.register(ZafepelConfig, ZafepelForCausalLM)
    except ValueError:                                                       # registered already
        pass


_register()
