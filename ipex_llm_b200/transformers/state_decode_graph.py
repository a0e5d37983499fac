"""One decode step of a model that keeps a ``DynamicStateCache`` (windowed attention + recurrent states), recorded in a CUDA
graph, and the greedy ``generate`` that replays it -- the counterpart of ``decode_graph.py`` (which records a llama-family
step against an FP8 key/value arena) for models whose forward this package owns.

What is recorded is the model's own forward for one new token per row, the pick of the next token and its write into the
step's input: nothing runs on the host between tokens.  A graph holds addresses, so the step owns its cache
(``frozen``: storage sized once for prompt + new tokens, never trimmed or moved; the convolution tails shifted in place; the
padding written into the same tensor) and everything that changes from token to token lives in device memory: the number of
positions each attention layer holds (``lengths``, read by the kernels instead of their host argument), the step counter,
the token.  ``generate()`` requests that are plain greedy decoding take this path; everything else (sampling, beams,
processors, streamers) goes to transformers' ``generate`` on the same forward, and both produce the same tokens.
"""
import copy
import os
import time
from collections import OrderedDict

import torch

from ipex_llm_b200.transformers.cuda_graph import capture_decode_step
from ipex_llm_b200.transformers.kv import DynamicStateCache

MAX_BATCH = 64
CAPACITY_STEP = 256           # total lengths are rounded up to this many positions (one recorded step per batch and capacity)
MAX_GRAPHS = 4


class StateDecodeGraph:
    def __init__(self, model, batch, capacity):
        self.model, self.B, self.capacity = model, batch, capacity
        dev = model.get_input_embeddings().weight.device
        self.device = dev
        self.cache = DynamicStateCache(reserve=capacity)
        self.cache.frozen = True
        self.ids = torch.zeros(batch, 1, dtype=torch.int64, device=dev)
        self.tokens = torch.zeros(batch, capacity, dtype=torch.int64, device=dev)
        self.step_index = torch.zeros(1, dtype=torch.int64, device=dev)
        with torch.no_grad(), torch.cuda.device(dev):
            # a two-token prompt allocates every state at its final size and address; then the step is run and recorded
            model(input_ids=torch.zeros(batch, 2, dtype=torch.int64, device=dev), past_key_values=self.cache, use_cache=True, logits_to_keep=1)
            kvs = [l.kv for l in self.cache.layers if l is not None and l.kv is not None]
            self.lengths = torch.zeros(max(len(kvs), 1), dtype=torch.int32, device=dev)
            for i, kv in enumerate(kvs):
                kv.length_dev = self.lengths[i:i + 1]
            self.kvs = kvs
            self._sync_lengths()
            torch.cuda.synchronize(dev)                  # the recording runs on a stream of its own
            self.graph = capture_decode_step(self._step, warmup=2)
        torch.cuda.current_stream(dev).wait_stream(self.graph.stream)

    def _sync_lengths(self):
        self.lengths.copy_(torch.tensor([kv.get_seq_length() for kv in self.kvs] or [0], dtype=torch.int32))

    def _step(self):
        out = self.model(input_ids=self.ids, past_key_values=self.cache, use_cache=True, logits_to_keep=1)
        nxt = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)              # [B, 1]
        self.tokens.index_copy_(1, self.step_index, nxt)
        self.ids.copy_(nxt)
        self.step_index.add_(1)
        self.lengths.add_(1)
        return self.tokens

    def run(self, input_ids, attention_mask, max_new):
        """prefill through the model's forward into the step's own cache, then max_new - 1 replays; returns [B, max_new]"""
        dev = self.device
        self.cache.restart()
        self.lengths.zero_()
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, past_key_values=self.cache, use_cache=True, logits_to_keep=1)
        first = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
        self.tokens[:, 0:1] = first
        self.ids.copy_(first)
        self.step_index.fill_(1)
        self._sync_lengths()
        stream = self.graph.stream
        stream.wait_stream(torch.cuda.current_stream(dev))
        for _ in range(max_new - 1):
            self.graph.replay()
        torch.cuda.current_stream(dev).wait_stream(stream)
        return self.tokens[:, :max_new].clone()


def _capacity_for(total_len):
    return max(2 * CAPACITY_STEP, -(-total_len // CAPACITY_STEP) * CAPACITY_STEP)


def get_state_graph(model, batch, total_len):
    graphs = model.__dict__.setdefault("_b200_state_graphs", OrderedDict())
    w = model.get_input_embeddings().weight
    key = (batch, _capacity_for(total_len), w.device, w.dtype)
    g = graphs.get(key)
    if g is None:
        while len(graphs) >= MAX_GRAPHS:
            graphs.popitem(last=False)
        g = graphs[key] = StateDecodeGraph(model, batch, key[1])
    else:
        graphs.move_to_end(key)
    return g


_PLAIN_KEYS = {"input_ids", "attention_mask", "max_new_tokens", "min_new_tokens", "max_length", "do_sample", "num_beams", "eos_token_id",
               "pad_token_id", "use_cache", "temperature", "top_p", "top_k"}


def _plan(model, inputs, generation_config, kwargs):
    """(input_ids, attention_mask, max_new, min_new, eos ids, pad id) if the recorded step serves the request, else None"""
    if os.environ.get("IPEX_LLM_B200_DECODE_GRAPH", "1") == "0" or not torch.cuda.is_available():
        return None
    if any(k not in _PLAIN_KEYS for k in kwargs):
        return None
    input_ids = kwargs.get("input_ids", inputs)
    w = model.get_input_embeddings().weight
    if not (torch.is_tensor(input_ids) and input_ids.dim() == 2 and input_ids.dtype == torch.int64 and input_ids.device == w.device
            and w.device.type == "cuda" and 1 <= input_ids.shape[0] <= MAX_BATCH and input_ids.shape[1] >= 1):
        return None
    gc = copy.deepcopy(generation_config if generation_config is not None else model.generation_config)
    gc.update(**{k: v for k, v in kwargs.items() if k not in ("input_ids", "attention_mask")})
    plain = (not gc.do_sample and (gc.num_beams or 1) == 1 and (gc.repetition_penalty or 1.0) == 1.0 and not gc.no_repeat_ngram_size
             and not gc.bad_words_ids and (gc.num_return_sequences or 1) == 1 and not gc.output_scores
             and not getattr(gc, "output_logits", False) and not gc.return_dict_in_generate and not gc.output_attentions
             and not gc.output_hidden_states and not getattr(gc, "suppress_tokens", None)
             and not getattr(gc, "begin_suppress_tokens", None) and not getattr(gc, "sequence_bias", None)
             and getattr(gc, "forced_eos_token_id", None) is None and not getattr(gc, "stop_strings", None)
             and not getattr(gc, "max_time", None) and gc.use_cache is not False and not (gc.min_new_tokens or 0) and not gc.min_length)
    if not plain:
        return None
    prompt_len = input_ids.shape[1]
    max_new = gc.max_new_tokens if gc.max_new_tokens is not None else (gc.max_length or 20) - prompt_len
    if max_new < 1:
        return None
    eos = gc.eos_token_id
    eos = [] if eos is None else ([int(eos)] if not isinstance(eos, (list, tuple)) else [int(e) for e in eos])
    pad = gc.pad_token_id if gc.pad_token_id is not None else (eos[0] if eos else 0)
    return input_ids, kwargs.get("attention_mask"), max_new, eos, pad


@torch.no_grad()
def generate_greedy_state_graph(self, inputs=None, generation_config=None, **kwargs):
    """``generate`` of a model with a ``DynamicStateCache``: plain greedy requests replay the recorded step"""
    plan = _plan(self, inputs, generation_config, kwargs)
    if plan is None:
        return self._hf_generate(inputs, generation_config=generation_config, **kwargs)
    input_ids, attention_mask, max_new, eos, pad = plan
    B, prompt_len = input_ids.shape
    dev = input_ids.device
    with torch.cuda.device(dev):
        try:
            g = None if self.__dict__.get("_b200_state_graph_failed") else get_state_graph(self, B, prompt_len + max_new)
        except RuntimeError as e:                            # a step that cannot be recorded: transformers' loop serves the model
            self.__dict__["_b200_state_graph_failed"] = str(e)
            g = None
        if g is None:
            return self._hf_generate(inputs, generation_config=generation_config, **kwargs)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        new_tokens = g.run(input_ids, attention_mask, max_new)
        torch.cuda.synchronize(dev)
        self.last_generate_seconds = time.perf_counter() - t0
    if eos:
        # rows that met an end-of-sequence token are padded behind it, and the result ends where the last row ended
        is_eos = torch.isin(new_tokens, torch.tensor(eos, device=dev))
        after = (is_eos.cumsum(1) - is_eos.to(torch.int64)) > 0
        new_tokens = new_tokens.masked_fill(after, pad)
        done = is_eos.any(dim=1)
        if bool(done.all()):
            new_tokens = new_tokens[:, :int((is_eos.to(torch.int64).argmax(dim=1)).max()) + 1]
    return torch.cat([input_ids, new_tokens], dim=1)


def install_state_generate(model):
    if getattr(model, "_hf_generate", None) is None:
        model._hf_generate = model.generate
        model.generate = generate_greedy_state_graph.__get__(model, model.__class__)
    return model
