"""Command line for the models of the registry (a folder with config.json + model.safetensors): token ids in, token ids out.

    python -m simplellminference_b200.generate --model DIR --prompt 5,17,3 --prompt 9,2 --max-new-tokens 32 [--dtype bfloat16|float32]
                                               [--temperature T --top-k K --top-p P --seed S] [--tokenizer spm.model --text "..."]

Every prompt is one request of a continuous batch (scheduler.ContinuousBatcher over seqengine.SequenceDecoder): prompts are taken in
portions beside the requests that already decode, each request keeps its own pages and state slot, next tokens are the first maximum of
the logits or, with --temperature, drawn on the device. With --tokenizer, --text prompts are encoded and the results decoded by the
sentencepiece model (predict.SPELayer), as the one-sequence driver does (reference source/model/model.cpp:142-187)."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--prompt", action="append", default=[], help="comma-separated token ids (repeatable)")
    ap.add_argument("--text", action="append", default=[], help="text prompt (needs --tokenizer; repeatable)")
    ap.add_argument("--tokenizer", help="sentencepiece model file")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--max-seqs", type=int, default=4)
    ap.add_argument("--max-tokens", type=int, default=0, help="positions the cache pool holds (0 = enough for every request at once)")
    ap.add_argument("--prefill-chunk", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--eos", type=int, default=None)
    a = ap.parse_args(argv)

    import torch
    if not torch.cuda.is_available():
        print("generate needs a CUDA device: this framework has no CPU path", file=sys.stderr)
        return 2
    from .models import build_model
    from .scheduler import ContinuousBatcher
    from .seqengine import SequenceDecoder, SequenceEngine

    spe = None
    if a.tokenizer:
        from .predict import SPELayer
        spe = SPELayer(a.tokenizer)
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt]
    if a.text:
        if spe is None:
            ap.error("--text needs --tokenizer")
        prompts += [spe.encode(t) for t in a.text]
    if not prompts:
        ap.error("give at least one --prompt or --text")
    model = build_model(a.model, a.dtype, "cuda", build=True)
    page_len = 64
    need = sum(-(-(len(p) + a.max_new_tokens) // page_len) * page_len for p in prompts)
    engine = SequenceEngine(model, max_tokens=a.max_tokens or need, max_seqs=a.max_seqs, page_len=page_len)
    cb = ContinuousBatcher(SequenceDecoder(engine, prefill_chunk=a.prefill_chunk), eos_id=a.eos)
    sampling = dict(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed) if a.temperature > 0 else None
    ids = [cb.submit(p, a.max_new_tokens, sampling) for p in prompts]
    out = cb.run()
    for rid, p in zip(ids, prompts):
        new = [int(t) for t in out[rid][len(p) - 1:]]
        rec = {"prompt": p, "tokens": new}
        if spe is not None:
            rec["text"] = spe.decode(new)
        print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
