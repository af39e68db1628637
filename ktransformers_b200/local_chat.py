"""Command line: load a checkpoint directory through the model registry and generate from token ids.

    python -m ktransformers_b200.local_chat --model_path DIR --prompt_ids 5,17,3 [--prompt_ids ...] --max_new_tokens 32
                                            [--dtype bfloat16|float32] [--temperature T --top_k K --top_p P --seed S]

(The reference's local_chat.py:56-170 does the same around a tokenizer and a chat template; the checkpoints served here
ship no tokenizer, so prompts are lists of ids and the output is one JSON line per prompt.)"""
from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model_path", required=True)
    ap.add_argument("--prompt_ids", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    ap.add_argument("--max_new_tokens", type=int, default=32)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top_k", type=int, default=0)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--max_tokens", type=int, default=8192, help="cache capacity in tokens")
    ap.add_argument("--chunk_size", type=int, default=2048, help="token budget of one step")
    a = ap.parse_args(argv)
    from .models import load_model
    from .util.engine import Engine, Sampler
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt_ids]
    model = load_model(a.model_path, a.dtype)
    eng = Engine(model, max_tokens=a.max_tokens, max_slots=max(8, len(prompts)), max_step_tokens=a.chunk_size)
    outs = eng.generate(prompts, a.max_new_tokens, Sampler(a.temperature, a.top_k, a.top_p, a.seed))
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt": p, "output": o}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
