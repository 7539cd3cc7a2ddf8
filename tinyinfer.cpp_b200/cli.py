"""Command line in the reference's manner (src/main.cpp:136-158, report at :300-310).

    python -m tinyinfer_b200.cli -m MODEL -n 128 -p "text" [-p ...] [-f prompts.txt]
        [-t temp] [--top-k K] [--top-p P] [--seed S] [--max-seq N] [--cuda-graph] [--verbose] [--chat]

Options keep the reference's names, meanings and defaults: ``-m`` model (a folder with
config.json and model.safetensors, or a GGUF file as the reference takes), ``-n`` new tokens
per prompt (128), ``-p`` a prompt (repeatable), ``-f`` a file with one prompt per non-empty
line, ``-t`` temperature (0 = greedy), ``--top-k`` (0 = off), ``--top-p`` (1.0), ``--seed`` (42),
``--max-seq`` context per request (2048), ``--cuda-graph`` replay steps from CUDA graphs,
``--verbose``, ``--chat`` (wrap each prompt in the Qwen3 chat form with an empty think block).

The engine works on token ids.  A prompt is text if the model brings a tokenizer (a GGUF file's
``tokenizer.ggml.*`` metadata, a folder's ``tokenizer.json``; read by this package's own
byte-level BPE tokenizer); otherwise, and always with ``--tokens``, it is a list of token ids
separated by spaces or commas.  Added options: ``--tokens``, ``--dtype``, ``--chunk``,
``--max-batched-tokens``, ``--max-num-seqs``, ``--page-size``, ``--kv-tokens``, and
``--random-weights CONFIG.json`` to run a configuration with seeded random weights.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def read_prompts_file(path: str) -> list[str]:
    """One prompt per non-empty line, carriage returns stripped (src/main.cpp:96-105)."""
    with open(path, "r", encoding="utf-8") as fh:
        return [ln.rstrip("\r\n") for ln in fh if ln.strip("\r\n")]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tinyinfer", description=__doc__,
                                 formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("-m", dest="model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-n", dest="n_predict", type=int, default=128)
    ap.add_argument("-p", dest="prompts", action="append", default=[])
    ap.add_argument("-f", dest="prompt_file")
    ap.add_argument("-t", dest="temp", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--max-seq", type=int, default=2048)
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--chat", action="store_true", help="wrap prompts in the Qwen3 chat form")
    ap.add_argument("--tokens", action="store_true", help="prompts are token ids, also when the model has a tokenizer")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--chunk", type=int, default=None, help="longest prompt portion per step")
    ap.add_argument("--max-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-num-seqs", type=int, default=16)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--kv-tokens", type=int, default=None, help="tokens the cache pool holds")
    ap.add_argument("--random-weights", metavar="CONFIG.json",
                    help="run this configuration with random weights drawn from --seed")
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    prompts = list(args.prompts)
    if args.prompt_file:
        try:
            prompts += read_prompts_file(args.prompt_file)
        except OSError:
            print(f"main: cannot read prompts file {args.prompt_file}", file=sys.stderr)
            return 1
    if (not args.model and not args.random_weights) or not prompts:
        ap.print_usage(sys.stderr)
        return 1

    from . import LLM, SamplingParams

    from .tokenizer import Tokenizer, TokenizerError, chat_wrap
    tokenizer = None
    if args.model and not args.tokens:
        try:
            tokenizer = Tokenizer.for_model(args.model)
        except (TokenizerError, OSError, ValueError) as exc:
            print(f"main: cannot read the model's tokenizer: {exc}", file=sys.stderr)
            return 1
    token_lists = []
    for s, text in enumerate(prompts):
        if tokenizer is not None:
            ids = tokenizer.encode(chat_wrap(text) if args.chat else text, parse_special=args.chat)
        else:
            try:
                ids = [int(x) for x in text.replace(",", " ").split()]
            except ValueError:
                print("main: the model brings no tokenizer; give prompts as token ids", file=sys.stderr)
                return 1
        if args.verbose:
            print(f"prompt {s} tokens: {len(ids)}", file=sys.stderr)
        token_lists.append(ids)
    if sum(len(t) for t in token_lists) == 0:
        print("main: empty prompts", file=sys.stderr)
        return 1

    kwargs = dict(dtype=args.dtype, max_seq=args.max_seq, max_num_seqs=args.max_num_seqs,
                  max_batched_tokens=args.max_batched_tokens, chunk=args.chunk,
                  page_size=args.page_size, kv_tokens=args.kv_tokens, cuda_graph=args.cuda_graph)
    if args.random_weights:
        with open(args.random_weights, "r", encoding="utf-8") as fh:
            llm = LLM(config=json.load(fh), seed=args.seed, **kwargs)
    else:
        llm = LLM(args.model, **kwargs)
    stop = () if tokenizer is None or tokenizer.eos_token_id is None else (tokenizer.eos_token_id,)
    params = SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p,
                            seed=args.seed, max_tokens=args.n_predict, stop_token_ids=stop)
    t0 = time.perf_counter()
    outs = llm.generate(token_lists, params, log_steps=args.verbose)
    seconds = time.perf_counter() - t0
    for s, (text, gen) in enumerate(zip(prompts, outs)):
        print(f"==================== prompt {s} ====================")
        print(f"[prompt] {text}")
        made = gen.tokens[:-1] if gen.finish_reason == "stop" and tokenizer else gen.tokens
        shown = tokenizer.decode(made) if tokenizer else " ".join(map(str, gen.tokens))
        print(f"[output] {shown}")
    st = llm.stats
    print(f"main: {st.steps} steps, {st.prompt_tokens} prompt tokens, {st.decode_tokens} decode "
          f"tokens, {st.preemptions} preemptions", file=sys.stderr)
    print(f"main: {seconds * 1e3:.1f} ms, {st.generated} tokens, "
          f"{st.generated / max(seconds, 1e-9):.1f} tok/s "
          f"[cuda-graph: {'on' if args.cuda_graph else 'off'}]", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
