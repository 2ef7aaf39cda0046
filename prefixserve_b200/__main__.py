"""Command line: offline generation from token ids.

    python -m prefixserve_b200 --model DIR --prompt-ids 1,2,3 --max-tokens 16

Option names and meanings follow the reference's command line where it has
them (prefixserve/server.py:567-581): --model, --dtype, --max-seq-len,
--num-blocks, --max-waiting, --max-running-requests, --chunked-prefill-size
(both the per-step budget and the longest portion), --disable-prefix-cache.
The reference serves HTTP and tokenises text; this program reads token ids and
prints token ids (one JSON object per prompt, then the scheduler's counters).
Without --model, --random-config NAME --seed N first writes a random-weights
model folder and runs that.  --max-seq-len defaults to the smaller of the
reference's 8192 and the model's own position limit.

Two sub-commands hand over to the other programs of the repository:
``python -m prefixserve_b200 replay ...`` is ``bin/trace_run ...`` and
``python -m prefixserve_b200 bench ...`` is ``bench.py ...`` of a source checkout.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="python -m prefixserve_b200", description="B200 Llama engine: offline generation")
    p.add_argument("--model", default=None, help="model folder (config.json, model.safetensors)")
    p.add_argument("--random-config", default=None, help="write and run a random-weights model of this preset")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    p.add_argument("--save-model", default=None, help="with --random-config: keep the written folder here")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--max-seq-len", type=int, default=None, help="default: min(8192, the model's max_position_embeddings)")
    p.add_argument("--num-blocks", type=int, default=None, help="cache pages; default: sized from free GPU memory")
    p.add_argument("--max-waiting", type=int, default=1024)
    p.add_argument("--max-running-requests", type=int, default=64)
    p.add_argument("--chunked-prefill-size", type=int, default=512)
    p.add_argument("--disable-prefix-cache", action="store_true")
    p.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; may be repeated")
    p.add_argument("--prompt-file", default=None, help="file with one prompt per line (comma- or space-separated ids)")
    p.add_argument("--max-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--sampling-seed", type=int, default=0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--stop-token-ids", default="", help="comma-separated ids that end a request, beside the model's own")
    p.add_argument("--cast-float32-weights", action="store_true",
                   help="round matrices the checkpoint stores in 32-bit to the compute type at load (the reference does)")
    return p.parse_args(argv)


def read_prompts(args: argparse.Namespace) -> list[list[int]]:
    lines = list(args.prompt_ids)
    if args.prompt_file:
        lines += [ln for ln in Path(args.prompt_file).read_text().splitlines() if ln.strip()]
    prompts = [[int(t) for t in ln.replace(",", " ").split()] for ln in lines]
    if not prompts:
        raise SystemExit("give at least one prompt with --prompt-ids or --prompt-file")
    return prompts


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        import runpy
        script = Path(__file__).resolve().parents[1] / "bench.py"
        if not script.exists():
            raise SystemExit("bench.py lies beside the package in a source checkout; it is not part of an installed package")
        sys.argv = [str(script)] + argv[1:]
        runpy.run_path(str(script), run_name="__main__")
        return 0
    args = parse_args(argv)
    prompts = read_prompts(args)
    if (args.model is None) == (args.random_config is None):
        raise SystemExit("give exactly one of --model and --random-config")

    import torch

    from .config.presets import preset
    from .engine.llm import LLM
    from .sampling import SamplingParams
    from .weights import write_random_model

    holder = None
    model_dir = args.model
    if model_dir is None:
        cfg = preset(args.random_config)
        if args.save_model:
            model_dir = args.save_model
        else:
            holder = tempfile.TemporaryDirectory(prefix="psb200-model-")
            model_dir = holder.name
        write_random_model(model_dir, cfg, args.seed, dtype=torch.bfloat16)
    try:
        llm = LLM(model_dir, dtype=args.dtype, max_seq_len=args.max_seq_len, num_blocks=args.num_blocks,
                  max_running_requests=args.max_running_requests, chunked_prefill_size=args.chunked_prefill_size,
                  enable_prefix_cache=not args.disable_prefix_cache, max_waiting=args.max_waiting,
                  cast_float32_weights=args.cast_float32_weights)
        stops = tuple(int(t) for t in args.stop_token_ids.replace(",", " ").split())
        sp = SamplingParams(temperature=args.temperature, seed=args.sampling_seed, max_tokens=args.max_tokens,
                            ignore_eos=args.ignore_eos, stop_token_ids=stops)
        outputs = llm.generate(prompts, sp)
        for prompt, out in zip(prompts, outputs):
            print(json.dumps({"prompt_ids": prompt, "output_ids": out}))
        st = llm.stats()
        print(json.dumps({"stats": {k: getattr(st, k) for k in st.__dataclass_fields__}, "prefix_hit_rate": st.prefix_hit_rate}))
    finally:
        if holder is not None:
            holder.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
