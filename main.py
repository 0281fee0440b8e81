"""Command line of the engine, in the manner of the reference's ``main.py``.

The reference keeps its knobs as constants at the top of ``main()``
(main.py:17-27: model_name_or_path, max_new_tokens, max_num_seqs,
max_model_len, block_size, num_blocks, dtype by device) and serves three demo
prompts.  Here the same names are options with the same meanings and
defaults; prompts come as text (needs tokenizer files in the model folder) or
as token ids.

    python main.py --model-name-or-path DIR --prompt-ids 1,2,3 --max-new-tokens 64
    python main.py --random-weights tiny-a --prompt-ids 5,6,7 --prompt-ids 9,9
"""
from __future__ import annotations

import argparse
import sys
import tempfile


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Qwen3 dense inference on one B200")
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model-name-or-path", "--model", dest="model", help="folder with config.json and model.safetensors")
    src.add_argument("--random-weights", metavar="PRESET", help="a named configuration with seeded random weights "
                     "(tiny-a, tiny-b, qwen3-0.6b, qwen3-1.7b, qwen3-4b)")
    ap.add_argument("--seed", type=int, default=None, help="seed of the random weights (default: the preset's)")
    ap.add_argument("--write-model", metavar="DIR", help="with --random-weights: write the model folder here and exit")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--prompt", action="append", default=[], help="a text prompt (repeatable)")
    ap.add_argument("--prompt-ids", action="append", default=[], help="a prompt as comma-separated token ids (repeatable)")
    ap.add_argument("--prompt-file", help="one prompt a line; lines of only numbers and commas are token ids")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--max-num-seqs", type=int, default=4)
    ap.add_argument("--max-model-len", type=int, default=256)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=None, help="default: max_num_seqs * ceil(max_model_len / block_size)")
    ap.add_argument("--gpu-memory-fraction", type=float, default=None,
                    help="without --num-blocks: size the cache from what this share of the device's memory leaves after the weights")
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=None, help="largest portion of a prompt in one step")
    ap.add_argument("--no-prefix-cache", action="store_true")
    ap.add_argument("--no-run-ahead", action="store_true",
                    help="do not launch a decode step before the host has read the tokens of the step before it")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--sample-seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--stats", action="store_true", help="print the engine's counters at the end")
    ap.add_argument("--profile", action="store_true",
                    help="time every step on the device and print steps, tokens and device time by kind of step "
                         "(prompt portions, decoded tokens, mixed) at the end")
    return ap


def _parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(" ", "").split(",") if t]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch
    from qwen_engine_b200 import LLM, SamplingParams
    from qwen_engine_b200.config import parse_dtype, preset_config_dict, preset_init
    from qwen_engine_b200.registry import config_from_dict
    from qwen_engine_b200.weights import write_model_folder

    block_size = args.block_size
    model = args.model
    if args.random_weights:
        cfg = config_from_dict(preset_config_dict(args.random_weights))
        init = preset_init(args.random_weights)
        seed = init["seed"] if args.seed is None else args.seed
        target = args.write_model or tempfile.mkdtemp(prefix="qwen_engine_b200_model_")
        write_model_folder(cfg, target, seed, init["std"], init["norm_std"])
        if args.write_model:
            print(f"wrote {target}")
            return 0
        model = target

    prompts: list = list(args.prompt) + [_parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line:
                    prompts.append(_parse_ids(line) if all(c.isdigit() or c in ", " for c in line) else line)
    if not prompts:
        print("no prompt given (--prompt, --prompt-ids or --prompt-file)", file=sys.stderr)
        return 2

    llm = LLM(model, dtype=parse_dtype(args.dtype), device=args.device, block_size=block_size,
              num_blocks=args.num_blocks, gpu_memory_fraction=args.gpu_memory_fraction, max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens, prefill_chunk_size=args.prefill_chunk,
              enable_prefix_cache=not args.no_prefix_cache, run_ahead=not args.no_run_ahead, seed=args.sample_seed,
              profile=args.profile)
    sp = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
                        seed=args.sample_seed, ignore_eos=args.ignore_eos)

    def print_info(prompt_text, output_text):       # the reference's print_info (main.py:74-79)
        print("=" * 88)
        print(f"Prompt: {prompt_text}")
        print("=" * 88)
        print(output_text)
        print("=" * 88)

    llm.engine.submit(prompts, sampling=sp)
    llm.engine.serving(print_func=print_info)
    torch.cuda.synchronize()
    if args.stats:
        print(llm.stats())
    if args.profile:
        print(llm.stats().profile_table())
    return 0


if __name__ == "__main__":
    sys.exit(main())
