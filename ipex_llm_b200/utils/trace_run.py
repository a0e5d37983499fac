"""Replay a trace of token steps through a model and write the logits the trace asks for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR [--max-tokens N] [--low-bit QTYPE]

The model is loaded the way every user of the package loads one (``AutoModelForCausalLM.from_pretrained``, which picks the
model class by config.json) and driven through the forward that ``generate()`` drives, with the cache that forward picks;
nothing is sampled.  Steps arrive on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: per request its next tokens and the places among them whose logits are wanted; ``end``: requests that are over
after this step (their rows leave the batch, their cache is released).  The entries of a step form one batch: either all of
them start (a new batch: rows are left-padded to the longest, as ``generate()`` pads) or all of them continue the batch they
started in.  For a step that wants something, ``<out>/<step>.f32`` receives the wanted rows as little-endian float32
[wanted, vocab], in the order of the entries and of ``want``; every step is answered by a line ``done <step>``.
"""
import argparse
import json
import os
import sys

import torch


class Batch:
    """requests that started together: their rows in the cache, in order"""

    def __init__(self, ids, cache):
        self.ids, self.cache = list(ids), cache

    def drop(self, gone):
        keep = [i for i, r in enumerate(self.ids) if r not in gone]
        if len(keep) != len(self.ids):
            self.ids = [self.ids[i] for i in keep]
            if keep:
                self.cache.batch_select_indices(torch.tensor(keep, dtype=torch.int64))


class Replayer:
    def __init__(self, model, device):
        self.model, self.device = model, device
        self.batch_of = {}                                   # request id -> Batch

    @torch.no_grad()
    def step(self, entries):
        """returns float32 [wanted, vocab] (or None)"""
        if not entries:
            return None
        ids = [e["id"] for e in entries]
        new = [r not in self.batch_of for r in ids]
        lengths = [len(e["tokens"]) for e in entries]
        width = max(lengths)
        tokens = torch.zeros(len(entries), width, dtype=torch.int64)
        mask = torch.zeros(len(entries), width, dtype=torch.int64)
        for i, e in enumerate(entries):
            tokens[i, width - lengths[i]:] = torch.tensor(e["tokens"], dtype=torch.int64)
            mask[i, width - lengths[i]:] = 1
        if all(new):
            batch = Batch(ids, None)
            for r in ids:
                self.batch_of[r] = batch
            kwargs = {"attention_mask": mask.to(self.device), "past_key_values": None}
        else:
            if any(new):
                raise ValueError("a step either starts requests or continues them")
            batch = self.batch_of[ids[0]]
            if any(self.batch_of[r] is not batch for r in ids) or min(lengths) != width:
                raise ValueError("the requests of a step continue one batch, by the same number of tokens")
            batch.drop(set(batch.ids) - set(ids))            # rows that sit this step out have ended
            if batch.ids != ids:
                order = [batch.ids.index(r) for r in ids]
                batch.cache.batch_select_indices(torch.tensor(order, dtype=torch.int64))
                batch.ids = ids
            kwargs = {"attention_mask": None, "past_key_values": batch.cache}
        wanted = [(i, width - lengths[i] + w) for i, e in enumerate(entries) for w in e["want"]]
        places = sorted({p for _, p in wanted})
        keep = torch.tensor(places if places else [width - 1], dtype=torch.int64)
        out = self.model(input_ids=tokens.to(self.device), use_cache=True, logits_to_keep=keep.to(self.device), **kwargs)
        batch.cache = out.past_key_values
        if not wanted:
            return None
        col = {p: k for k, p in enumerate(places)}
        rows = torch.tensor([i for i, _ in wanted], dtype=torch.int64, device=out.logits.device)
        cols = torch.tensor([col[p] for _, p in wanted], dtype=torch.int64, device=out.logits.device)
        return out.logits[rows, cols].to(torch.float32).cpu()

    def end(self, ids):
        for r in ids:
            batch = self.batch_of.pop(r, None)
            if batch is not None:
                batch.drop({r})


def load(model_dir, dtype, low_bit=None):
    from ipex_llm_b200.transformers import AutoModelForCausalLM
    kwargs = {"torch_dtype": dtype}
    if low_bit:
        kwargs["load_in_low_bit"] = low_bit
    model = AutoModelForCausalLM.from_pretrained(model_dir, **kwargs)
    return model.eval()


def main(argv=None, stdin=None, stdout=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and the weights")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, default=0, help="most tokens live at a time (caches grow on demand; not needed)")
    ap.add_argument("--low-bit", default=None, help="convert the linears to this low-bit format first (e.g. sym_int4)")
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    dtype = getattr(torch, a.dtype)
    # 16-bit matrix products accumulate in 32 bits all the way (no 16-bit reduction between the parts of a split product)
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    if a.dtype == "float32":
        # true 32-bit: no TF32 in the matrix products
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
    if a.device.startswith("cuda") and not torch.cuda.is_available():
        print("trace_run: no CUDA device (the kernels have no CPU path)", file=sys.stderr)
        return 2
    device = torch.device(a.device)
    model = load(a.model, dtype, a.low_bit).to(device)
    os.makedirs(a.out, exist_ok=True)
    replayer = Replayer(model, device)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        logits = replayer.step(step.get("entries", []))
        if logits is not None:
            path = os.path.join(a.out, "%d.f32" % step["step"])
            with open(path + ".part", "wb") as f:
                f.write(logits.contiguous().numpy().astype("<f4").tobytes())
            os.replace(path + ".part", path)
        replayer.end(step.get("end", []))
        stdout.write("done %d\n" % step["step"])
        stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
