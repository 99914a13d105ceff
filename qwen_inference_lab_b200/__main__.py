"""python -m qwen_inference_lab_b200 --model DIR --token-ids '[1, 2, 3]' --dtype bfloat16

Options keep the reference's names and meanings where it has them
(qil/__main__.py:9-21): --model, --prompt | --token-ids, --dtype, --max-new-tokens,
--pages, --page-size, --chunk-size, --output.  --device accepts only cuda;
--sdpa-backend and --decode-attention have no counterpart (one attention path).
"""
import argparse
import json
import sys
from pathlib import Path


def build_parser():
    parser = argparse.ArgumentParser(prog="python -m qwen_inference_lab_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--prompt", help="text; needs the tokenizer files in --model and the transformers package")
    source.add_argument("--token-ids", help="JSON list of token ids")
    parser.add_argument("--device", default="cuda", choices=["cuda"])
    parser.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    parser.add_argument("--max-new-tokens", default=64, type=int)
    parser.add_argument("--pages", default=256, type=int)
    parser.add_argument("--page-size", default=16, type=int)
    parser.add_argument("--chunk-size", default=64, type=int, help="most prompt tokens of a request per step")
    parser.add_argument("--token-budget", default=128, type=int, help="most tokens per step over all requests")
    parser.add_argument("--max-active", default=4, type=int)
    parser.add_argument("--temperature", default=0.0, type=float, help="0 = greedy")
    parser.add_argument("--seed", default=0, type=int, help="sampling seed")
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--random-weights", type=int, metavar="SEED", default=None,
                        help="write model.safetensors with random weights for --model's config.json first")
    parser.add_argument("--output", type=Path)
    return parser


def main(argv=None):
    args = build_parser().parse_args(argv)
    from . import models  # noqa: F401
    from .config import registry
    from .engine.engine import Engine
    from .loading import load_model
    from .weights import write_model_folder

    if args.random_weights is not None:
        _, config = registry.read_model_config(args.model)
        write_model_folder(config, args.random_weights, args.model)
    tokenizer = None
    if args.prompt is not None:
        from transformers import AutoTokenizer   # tokenizer only; no model code of that package is used
        tokenizer = AutoTokenizer.from_pretrained(args.model, local_files_only=True)
        tokens = tokenizer.encode(args.prompt, add_special_tokens=False)
    else:
        tokens = json.loads(args.token_ids)
    model = load_model(args.model, device=args.device, dtype=args.dtype)
    engine = Engine(model, num_pages=args.pages, page_size=args.page_size, prefill_chunk=args.chunk_size,
                    token_budget=args.token_budget, max_active=args.max_active, seed=args.seed)
    try:
        result = engine.generate([tokens], max_new_tokens=args.max_new_tokens, ignore_eos=args.ignore_eos,
                                 temperature=args.temperature, seed=args.seed)[0]
        if tokenizer is not None:
            result["text"] = tokenizer.decode(result["token_ids"], skip_special_tokens=True)
        encoded = json.dumps(result, ensure_ascii=False, indent=2)
        if args.output:
            args.output.parent.mkdir(parents=True, exist_ok=True)
            args.output.write_text(encoded + "\n")
        print(encoded)
    finally:
        engine.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
