"""Command line of the engine, in the manner of the reference's `tiny_llama` program
(model/llm/tiny_llama.cpp:73-84): every line of standard input is one request, and
every finished request is printed as `<request id>: <output>`.  The reference takes
text and owns a tokenizer; here a line holds token ids (separated by spaces or
commas) and the output is the generated token ids.  End of input ends the program
once all requests are finished.

    python -m llm_b200 --model DIR [--dtype bfloat16] [--max-new-tokens 256] < prompts.txt
    python -m llm_b200 --model DIR --random-config config.json --random-seed 1   # writes DIR first
    python -m llm_b200 --model DIR --prompt-ids "1,2,3" --prompt-ids "7 8"       # requests from the command line
    python -m llm_b200 --model DIR --prompt-file prompts.txt                     # or from a file, one per line
"""
from __future__ import annotations

import argparse
import json
import select
import sys


def parse_line(line: str):
    return [int(x) for x in line.replace(",", " ").split()]


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m llm_b200", description=__doc__,
                                formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max-num-seqs", type=int, default=8)
    p.add_argument("--max-num-batched-tokens", type=int, default=512)
    p.add_argument("--max-seq-len", type=int, default=None)
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--eos-token-id", type=int, default=None, help="default: the model's; -1: never stop early")
    p.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    p.add_argument("--seed", type=int, default=0, help="seed of temperature sampling")
    p.add_argument("--kv-block-size", type=int, default=16)
    p.add_argument("--num-kv-blocks", type=int, default=None)
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--random-config", default=None,
                   help="a config.json: write a random-weights model into --model first")
    p.add_argument("--random-seed", type=int, default=0)
    p.add_argument("--prompt-ids", action="append", default=[],
                   help="a request's token ids (may be given several times); standard input is then not read")
    p.add_argument("--prompt-file", default=None, help="requests from this file instead of standard input, one per line")
    args = p.parse_args(argv)

    if args.random_config:
        from .weights.loader import write_random_model
        with open(args.random_config, "r", encoding="utf-8") as f:
            write_random_model(args.model, json.load(f), args.random_seed, args.dtype)

    from .engine.llm import LLM
    llm = LLM(args.model, dtype=args.dtype, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens, max_seq_len=args.max_seq_len,
              eos_token_id=args.eos_token_id, kv_block_size=args.kv_block_size,
              num_kv_blocks=args.num_kv_blocks, gpu_memory_utilization=args.gpu_memory_utilization,
              use_cuda_graphs=not args.no_cuda_graphs)

    given = None
    if args.prompt_ids or args.prompt_file:
        given = [parse_line(x) for x in args.prompt_ids]
        if args.prompt_file:
            with open(args.prompt_file, "r", encoding="utf-8") as f:
                given += [parse_line(line) for line in f if line.strip()]
        given.reverse()

    def receive(wait: bool):
        if given is not None:                   # all requests are known: hand them over one by one
            return given.pop() if given else None
        while True:
            if not wait and not select.select([sys.stdin], [], [], 0)[0]:
                return None
            line = sys.stdin.readline()
            if not line:
                return None
            if line.strip():
                return parse_line(line)

    def emit(request_id: int, tokens):
        print(f"{request_id}: {' '.join(str(t) for t in tokens)}", flush=True)

    llm.server(receive, emit, max_new_tokens=args.max_new_tokens, temperature=args.temperature, seed=args.seed)
    return 0


if __name__ == "__main__":
    sys.exit(main())
