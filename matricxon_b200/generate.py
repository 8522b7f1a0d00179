"""Command line in the manner of the reference's manual StarCoder2 check
(tools/manual_generate_check_starcoder2.py:20-51): load a model, generate from one prompt,
print what came out.

    python -m matricxon_b200.generate --model-dir DIR --prompt-ids 1,2,3 --num-predict 30

``--model-dir`` takes the place of ``--gguf-path`` (a folder with config.json and
model.safetensors); ``--num-predict`` (default 30) and ``--temperature`` (default 0.0, greedy)
keep the reference's names, defaults and meanings, and the seed is fixed to 0 as there
(tools/manual_generate_check_starcoder2.py:41-46). The engine works on token ids; text needs a
tokenizer, which is outside this engine, so the prompt is given as ids (``--prompt-ids``) or
drawn at random (``--prompt-len``). ``--random-config NAME`` runs without a model folder on
seeded random weights.
"""

from __future__ import annotations

import argparse
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="python -m matricxon_b200.generate", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--model-dir", help="folder with config.json and model.safetensors")
    source.add_argument("--random-config", help="a config.json to run with seeded random weights")
    parser.add_argument("--prompt", default=None,
                        help="text prompt (refused: this engine has no tokenizer; use --prompt-ids)")
    parser.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    parser.add_argument("--prompt-len", type=int, default=16, help="length of a random prompt")
    parser.add_argument("--num-predict", type=int, default=30)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=40)
    parser.add_argument("--top-p", type=float, default=0.9)
    parser.add_argument("--repeat-penalty", type=float, default=1.1)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--eos-token-id", type=int, action="append", default=[])
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-batched-tokens", type=int, default=2048)
    parser.add_argument("--prefill-chunk", type=int, default=512)
    return parser


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if args.prompt is not None:
        print("error: --prompt needs a tokenizer, which this engine does not contain; "
              "pass --prompt-ids", file=sys.stderr)
        return 2

    import json

    import torch

    from matricxon_b200 import ChatEngine, GenerationRequest, SamplingConfig
    from matricxon_b200.config.registry import config_from_dict, load_config
    from matricxon_b200.engine.core import build_model, load_model
    from matricxon_b200.weights.random_init import RandomSource, weight_specs_for

    if args.model_dir:
        config = load_config(args.model_dir)
        _, model = load_model(args.model_dir, dtype=args.dtype, device=args.device,
                              page_size=args.page_size)
    else:
        with open(args.random_config, "r", encoding="utf-8") as handle:
            config = config_from_dict(json.load(handle), args.random_config)
        source = RandomSource(weight_specs_for(config), args.seed, device=args.device)
        model = build_model(config, source, args.dtype, args.device, args.page_size)
    print(f"architecture: {type(config).architecture} ({type(config).model_type})")
    print(f"dtype:        {args.dtype}")

    if args.prompt_ids:
        prompt = [int(piece) for piece in args.prompt_ids.split(",") if piece.strip()]
    else:
        generator = torch.Generator().manual_seed(args.seed)
        prompt = torch.randint(0, config.vocab_size, (args.prompt_len,), generator=generator).tolist()

    num_ctx = len(prompt) + args.num_predict + 8
    engine = ChatEngine(model, eos_token_ids=set(args.eos_token_id), max_cache_tokens=num_ctx + 64,
                        max_active=1, max_batched_tokens=args.max_batched_tokens,
                        prefill_chunk=args.prefill_chunk, max_model_len=num_ctx)
    sampling = SamplingConfig(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                              repeat_penalty=args.repeat_penalty, num_ctx=num_ctx,
                              num_predict=args.num_predict, seed=args.seed)
    started = time.monotonic()
    result = engine.generate(GenerationRequest(input_ids=prompt, sampling=sampling))
    elapsed = time.monotonic() - started
    print(f"prompt ids:     {prompt}")
    print(f"finish_reason:  {result.finish_reason}")
    print(f"generated ids:  {result.token_ids}")
    print(f"{len(result.token_ids)} tokens in {elapsed:.3f}s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
