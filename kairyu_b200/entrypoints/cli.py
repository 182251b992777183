"""``kairyu-b200`` console entry point, in the reference's argparse-subcommand
manner (kairyu/entrypoints/cli.py:12-40 has ``serve`` and ``validate``; this
engine has no server, so its commands are the offline ones).

    kairyu-b200 generate MODEL --prompt-token-ids 1,2,3 [sampling flags]
    kairyu-b200 validate MODEL
    kairyu-b200 make-random CONFIG.json OUT --seed 0
    kairyu-b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl

Sampling flags are named as the ``SamplingParams`` fields are.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Optional, Sequence


def _build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="kairyu-b200", description="kairyu_b200 offline inference CLI")
    commands = parser.add_subparsers(dest="command", required=True)

    generate = commands.add_parser("generate", help="Generate from a model folder (config.json + safetensors).")
    generate.add_argument("model", type=Path, help="Path to the model folder")
    generate.add_argument("--prompt", action="append", default=[], help="A text prompt (needs tokenizer.json); repeatable")
    generate.add_argument("--prompt-token-ids", action="append", default=[], help="Comma-separated token ids; repeatable")
    generate.add_argument("--prompt-file", type=Path, default=None, help="JSON lines: a string or a list of token ids a line")
    generate.add_argument("--dtype", default="auto", choices=["auto", "bfloat16", "float32"])
    generate.add_argument("--device", default="cuda", help="Device of the model and cache (the kernels need a CUDA device)")
    generate.add_argument("--seed", type=int, default=None)
    generate.add_argument("--temperature", type=float, default=1.0)
    generate.add_argument("--top-p", type=float, default=1.0)
    generate.add_argument("--top-k", type=int, default=-1)
    generate.add_argument("--min-p", type=float, default=0.0)
    generate.add_argument("--presence-penalty", type=float, default=0.0)
    generate.add_argument("--frequency-penalty", type=float, default=0.0)
    generate.add_argument("--repetition-penalty", type=float, default=1.0)
    generate.add_argument("--max-tokens", type=int, default=16)
    generate.add_argument("--min-tokens", type=int, default=0)
    generate.add_argument("--n", type=int, default=1)
    generate.add_argument("--stop", action="append", default=[])
    generate.add_argument("--stop-token-ids", default="", help="Comma-separated token ids")
    generate.add_argument("--ignore-eos", action="store_true")
    generate.add_argument("--logprobs", type=int, default=None, help="Report each generated token's log-probability and this many of the most likely")
    generate.add_argument("--page-size", type=int, default=16)
    generate.add_argument("--num-pages", type=int, default=None)
    generate.add_argument("--max-num-batched-tokens", type=int, default=2048)
    generate.add_argument("--max-num-seqs", type=int, default=256)
    generate.add_argument("--max-model-len", type=int, default=None)
    generate.add_argument("--decode-mode", choices=["eager", "cuda_graph"], default=None)
    generate.add_argument("--pipeline-depth", type=int, choices=[1, 2], default=1, help="2: launch step N+1 while step N runs")
    generate.add_argument("--enable-prefix-caching", action="store_true", help="Share whole cache pages between requests whose tokens start the same way")

    validate = commands.add_parser("validate", help="Check a model folder against its architecture without a GPU.")
    validate.add_argument("model", type=Path, help="Path to the model folder")

    make_random = commands.add_parser("make-random", help="Write a model folder with seeded random weights.")
    make_random.add_argument("config", type=Path, help="Path to a config.json")
    make_random.add_argument("out", type=Path, help="Folder to write")
    make_random.add_argument("--seed", type=int, default=0)
    make_random.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])

    replay = commands.add_parser("replay", help="Trace replay (same as bin/trace_run).", add_help=False)
    replay.add_argument("rest", nargs=argparse.REMAINDER)
    return parser


def _ids(text: str) -> list[int]:
    return [int(part) for part in text.replace(" ", "").split(",") if part]


def _generate(args: argparse.Namespace) -> int:
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    prompts: list = [text for text in args.prompt]
    prompts += [TokensPrompt(tuple(_ids(text))) for text in args.prompt_token_ids]
    if args.prompt_file is not None:
        for line in args.prompt_file.read_text().splitlines():
            if line.strip():
                item = json.loads(line)
                prompts.append(item if isinstance(item, str) else TokensPrompt(tuple(item)))
    if not prompts:
        print("kairyu-b200 generate: give --prompt, --prompt-token-ids or --prompt-file", file=sys.stderr)
        return 2
    params = SamplingParams(
        n=args.n, presence_penalty=args.presence_penalty, frequency_penalty=args.frequency_penalty,
        repetition_penalty=args.repetition_penalty, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
        min_p=args.min_p, seed=args.seed, stop=args.stop or None, stop_token_ids=_ids(args.stop_token_ids) or None,
        max_tokens=args.max_tokens, min_tokens=args.min_tokens, ignore_eos=args.ignore_eos, logprobs=args.logprobs,
    )
    llm = LLM(
        str(args.model), dtype=args.dtype, device=args.device, page_size=args.page_size, num_pages=args.num_pages,
        max_num_batched_tokens=args.max_num_batched_tokens, max_num_seqs=args.max_num_seqs,
        max_model_len=args.max_model_len, decode_mode=args.decode_mode, pipeline_depth=args.pipeline_depth,
        enable_prefix_caching=args.enable_prefix_caching,
    )
    for output in llm.generate(prompts, params):
        print(
            json.dumps(
                {
                    "request_id": output.request_id,
                    "prompt_token_ids": list(output.prompt_token_ids),
                    "outputs": [
                        {
                            "index": c.index, "token_ids": list(c.token_ids), "text": c.text,
                            "finish_reason": c.finish_reason, "stop_reason": c.stop_reason,
                            **(
                                {}
                                if c.logprobs is None
                                else {
                                    "cumulative_logprob": c.cumulative_logprob,
                                    "logprobs": [{str(token): value for token, value in entry.items()} for entry in c.logprobs],
                                }
                            ),
                        }
                        for c in output.outputs
                    ],
                }
            )
        )
    return 0


def _validate(args: argparse.Namespace) -> int:
    from kairyu_b200.engine.engine import build_model
    import fnmatch

    from kairyu_b200.weights import CheckpointReader, WeightError, read_config
    from kairyu_b200.weights.loading import IGNORED_TENSORS

    try:
        config = read_config(args.model)
        model, parsed = build_model(config, dtype="bfloat16", device="meta")
        reader = CheckpointReader(args.model)
        specs = model.tensor_specs()
        missing = [s.name for s in specs if s.name not in reader and not (s.alias_of and s.alias_of in reader)]
        wrong = [
            (s.name, reader.shape(s.name), tuple(s.shape)) for s in specs if s.name in reader and reader.shape(s.name) != tuple(s.shape)
        ]
        known = {s.name for s in specs} | {s.alias_of for s in specs if s.alias_of}
        unexpected = [
            name for name in reader.names()
            if name not in known and not any(fnmatch.fnmatch(name, pattern) for pattern in IGNORED_TENSORS)
        ]
        if missing or wrong or unexpected:
            raise WeightError(str(args.model), missing, unexpected, wrong, [])
    except Exception as error:  # report, do not trace
        print(f"invalid: {error}")
        return 1
    print(f"valid: {parsed.architecture}, {parsed.num_hidden_layers} layers, {len(specs)} tensors")
    return 0


def main(argv: Optional[Sequence[str]] = None) -> None:
    args = _build_parser().parse_args(argv)
    if args.command == "generate":
        code = _generate(args)
    elif args.command == "validate":
        code = _validate(args)
    elif args.command == "make-random":
        from kairyu_b200.weights import write_random_model

        out = write_random_model(json.loads(args.config.read_text()), args.out, seed=args.seed, dtype=args.dtype)
        print(f"wrote {out}")
        code = 0
    else:
        from kairyu_b200.entrypoints.trace_run import main as replay_main

        code = replay_main(args.rest)
    if code:
        sys.exit(code)


if __name__ == "__main__":
    main()
