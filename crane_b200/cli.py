"""``crane``: generate from a model folder on the command line.

Options that the reference's binary has keep its names and meanings
(crane-serve/src/lib.rs:27-52): ``-m/--model-path``, ``--model-type``,
``-c/--max-concurrent``, ``--max-seq-len``, ``--gpu-memory-limit``.  Host, port
and file format belong to its server and quantised formats and are not here.
The rest set the engine (``--dtype``, ``--page-size``, ...) and the request.
Prompts are token ids; text prompts need ``tokenizer.json`` in the folder and
the ``tokenizers`` package.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="crane", description="Hunyuan Dense generation on one B200")
    ap.add_argument("-m", "--model-path", required=True,
                    help="folder with config.json (and safetensors unless --random-weights)")
    ap.add_argument("--model-type", default="auto", help="auto, or a registered architecture/alias")
    ap.add_argument("-c", "--max-concurrent", type=int, default=16)
    ap.add_argument("--max-seq-len", type=int, default=0, help="0: the model's limit")
    ap.add_argument("--gpu-memory-limit", default=None, help='"5G", "5120M", a fraction, or bytes')
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32", "bfloat16", "float32"])
    ap.add_argument("--random-weights", action="store_true",
                    help="ignore safetensors: draw weights from --seed for the folder's config.json")
    ap.add_argument("--seed", type=int, default=0)
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("--prompt-ids", help="comma-separated token ids; ';' separates several prompts")
    g.add_argument("--prompt-file", help="file with one prompt of comma- or space-separated ids a line")
    g.add_argument("--prompt", help="text (needs tokenizer.json)")
    ap.add_argument("--chat", action="store_true",
                    help="with --prompt: the text is a user message, put into the Hunyuan chat template")
    ap.add_argument("--system", default=None, help="with --chat: a system message before the user's")
    ap.add_argument("--max-new-tokens", type=int, default=245)
    ap.add_argument("--temperature", type=float, default=None, help="omit for greedy")
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--repeat-last-n", type=int, default=5)
    ap.add_argument("--eos-token-id", type=int, default=None)
    ap.add_argument("--sampling-seed", type=int, default=1024)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--num-pages", type=int, default=0)
    ap.add_argument("--max-batched-tokens", type=int, default=2048)
    ap.add_argument("--chunk-size", type=int, default=2048)
    ap.add_argument("--report-speed", action="store_true")
    ap.add_argument("--stream", action="store_true", help="print tokens as they are generated")
    ap.add_argument("--stats", action="store_true", help="print the engine's counters at the end")
    return ap


def _parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    from .generation import GenerationConfig, ModelForCausalLM, TokenStreamer

    tokenizer = None
    if args.prompt is not None:
        path = os.path.join(args.model_path, "tokenizer.json")
        if not os.path.isfile(path):
            print(f"Tokenizer not found at {path}; give --prompt-ids instead", file=sys.stderr)
            return 2
        from tokenizers import Tokenizer
        tokenizer = Tokenizer.from_file(path)
        text = args.prompt
        if args.chat:
            from .generation.chat import format_chat
            text = format_chat(text, args.system)
        prompts = [tokenizer.encode(text, add_special_tokens=True).ids]
    elif args.prompt_ids is not None:
        prompts = [_parse_ids(p) for p in args.prompt_ids.split(";") if p.strip()]
    else:
        with open(args.prompt_file) as f:
            prompts = [_parse_ids(l) for l in f if l.strip()]

    options = dict(page_size=args.page_size, num_pages=args.num_pages,
                   max_concurrent=args.max_concurrent, max_seq_len=args.max_seq_len,
                   gpu_memory_limit=args.gpu_memory_limit,
                   max_batched_tokens=max(args.max_batched_tokens, args.max_concurrent),
                   chunk_size=args.chunk_size)
    model = ModelForCausalLM.from_pretrained(args.model_path, args.dtype, args.model_type,
                                             random_weights=args.random_weights, seed=args.seed, **options)

    gen = GenerationConfig(max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                           top_p=args.top_p, top_k=args.top_k,
                           repetition_penalty=args.repetition_penalty,
                           repeat_last_n=args.repeat_last_n, eos_token_id=args.eos_token_id,
                           report_speed=args.report_speed, seed=args.sampling_seed)

    class Printer(TokenStreamer):
        def append(self, token_id: int) -> None:
            text = tokenizer.decode([token_id]) if tokenizer else f"{token_id} "
            print(text, end="", flush=True)

        def finalize(self) -> None:
            print(flush=True)

    if len(prompts) == 1:
        out = [model.generate(prompts[0], gen, Printer() if args.stream else None)]
    else:
        out = model.generate_batch(prompts, gen)
    if not args.stream:
        for p, toks in zip(prompts, out):
            new = toks[len(p):]
            print(tokenizer.decode(new) if tokenizer else ",".join(str(t) for t in new))
    if args.stats:
        print(json.dumps(model.stats()), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
