"""Command line in the manner of the reference's binary (src/main.rs, options in
src/server/mod.rs:706-904): the same names and meanings where the reference has them.

    python -m xinfer_b200 --m DIR --prompts "1,2,3|4,5,6" --max-tokens 32
    python -m xinfer_b200 --m DIR --batch 8 --prompt-len 128 --max-tokens 64 --ignore-eos
    python -m xinfer_b200 --random CONFIG.json --seed 0 --m DIR      (write a random-weight folder)

Prompts are token ids (``|`` between prompts as in the reference, ``,`` between ids); with
``--batch N`` one prompt is repeated N times (src/main.rs:103-115).  The run ends with the
reference's two figures: prompt tokens per second and decoded tokens per second
(src/main.rs:502-555).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="xinfer_b200", description="Qwen3 inference on one B200")
    ap.add_argument("--m", dest="model_id", help="model folder (config.json and model.safetensors)")
    ap.add_argument("--w", dest="weight_path", help="same as --m (the reference's older spelling)")
    ap.add_argument("--dtype", default="bf16", help="bf16 (default) or f32")
    ap.add_argument("--d", dest="device_ids", help="the GPU to run on, by index (the reference takes a list: one device here)")
    ap.add_argument("--cpu", action="store_true", help="refused: this engine has no CPU path")
    ap.add_argument("--prompts", help="token ids: '1,2,3|4,5,6' ('|' between prompts)")
    ap.add_argument("--batch", type=int, help="repeat one prompt this many times (batch performance test)")
    ap.add_argument("--prompt-len", type=int, help="make a prompt of this many seeded random token ids")
    ap.add_argument("--max-tokens", type=int, default=16384, help="most tokens generated per request")
    ap.add_argument("--ignore-eos", action="store_true", help="continue after the model emits an EOS token")
    ap.add_argument("--temperature", type=float)
    ap.add_argument("--top-k", type=int)
    ap.add_argument("--top-p", type=float)
    ap.add_argument("--frequency-penalty", type=float)
    ap.add_argument("--presence-penalty", type=float)
    ap.add_argument("--seed", type=int, help="seed for sampling (and for --random / --prompt-len)")
    ap.add_argument("--max-num-seqs", type=int, default=None, help="most requests running at once")
    ap.add_argument("--max-model-len", type=int, help="longest sequence (prompt plus output)")
    ap.add_argument("--kv-fraction", type=float, default=0.7, help="share of free GPU memory given to the cache")
    ap.add_argument("--prefill-chunk-size", type=int, default=8192, help="longest prompt portion in one step")
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192, help="most tokens in one step")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--num-blocks", type=int, help="cache pages (default: from --kv-fraction)")
    ap.add_argument("--disable-cuda-graph", action="store_true")
    ap.add_argument("--poison-freed-pages", action="store_true",
                    help="debug: fill every cache page that is given back with NaN before the next step")
    ap.add_argument("--disable-run-ahead", action="store_true",
                    help="wait for every step's tokens before the next step is decided")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="write a random-weight model folder to --m from this config and --seed, then exit")
    ap.add_argument("--store-dtype", default="bf16", help="dtype of the tensors --random writes (bf16 or f32)")
    return ap


def _parse_prompts(text: str) -> List[List[int]]:
    out = []
    for part in text.split("|"):
        ids = [int(x) for x in part.replace(" ", ",").split(",") if x != ""]
        if not ids:
            raise SystemExit("--prompts: an empty prompt")
        out.append(ids)
    return out


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.model_id and args.weight_path:
        raise SystemExit("use either --m or --w, not both")
    folder = args.model_id or args.weight_path
    if not folder:
        raise SystemExit("--m <model folder> is required")
    if args.cpu:
        raise SystemExit("--cpu: this engine runs on a B200 only; there is no CPU path")
    device = "cuda:0"
    if args.device_ids:
        ids = [x for x in args.device_ids.split(",") if x != ""]
        if len(ids) != 1 or not ids[0].isdigit():
            raise SystemExit(f"--d {args.device_ids}: this engine runs on one GPU; give one device index")
        device = f"cuda:{ids[0]}"
    if args.random:
        import torch
        from .weights import write_random_model
        with open(args.random) as f:
            cfg = json.load(f)
        store = torch.float32 if args.store_dtype in ("f32", "float32") else torch.bfloat16
        write_random_model(folder, cfg, args.seed or 0, dtype=store)
        print(f"wrote {folder}/config.json and model.safetensors (seed {args.seed or 0})")
        return 0

    import numpy as np
    from . import Engine, EngineConfig, GenerationConfig, SamplingParams
    from .config import load_config

    if args.prompts:
        prompts = _parse_prompts(args.prompts)
    else:
        _, cfg = load_config(folder)
        rng = np.random.default_rng(args.seed or 0)
        prompts = [rng.integers(0, cfg.vocab_size, size=args.prompt_len or 16).tolist()]
    if args.batch:
        prompts = [prompts[0]] * args.batch
    # sampling flags make the engine's default options, as in the reference (src/main.rs:117-135); they come
    # before those of the folder's generation_config.json
    flags = dict(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                 frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty)
    generation_cfg = GenerationConfig(**flags) if any(v is not None for v in flags.values()) else None
    econfig = EngineConfig(
        weight_path=folder, generation_cfg=generation_cfg, device=device, block_size=args.block_size, num_blocks=args.num_blocks,
        kv_fraction=args.kv_fraction, max_num_seqs=args.max_num_seqs or max(len(prompts), 1),
        max_num_batched_tokens=args.max_num_batched_tokens, prefill_chunk_size=args.prefill_chunk_size,
        max_model_len=args.max_model_len, max_tokens=args.max_tokens, seed=args.seed,
        disable_cuda_graph=args.disable_cuda_graph, disable_run_ahead=args.disable_run_ahead,
        poison_freed_pages=args.poison_freed_pages)
    t0 = time.time()
    engine = Engine(econfig, args.dtype)
    print(f"model loaded in {time.time() - t0:.1f} s; cache holds {engine.runner.kv_cache_tokens()} tokens", file=sys.stderr)
    params = SamplingParams(max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    outs = engine.generate_sync(params, prompts)
    for o in outs:
        print(f"[seq {o.seq_id}] prompt {o.prompt_length} tokens -> {o.decoded_length} tokens ({o.finish_reason}): "
              + ",".join(str(t) for t in o.decode_output))
    prompt_s = max(max(o.decode_start_time - o.prompt_start_time for o in outs) / 1000.0, 1e-6)
    decode_s = max(sum(o.decode_finish_time - o.decode_start_time for o in outs) / len(outs) / 1000.0, 1e-6)
    n_prompt = sum(o.prompt_length for o in outs)
    n_dec = sum(o.decoded_length for o in outs)
    print(f"Prompt tokens: {n_prompt} in {prompt_s:.2f}s ({n_prompt / prompt_s:.2f} tokens/s)")
    print(f"Decoded tokens: {n_dec} in {decode_s:.2f}s ({n_dec / decode_s:.2f} tokens/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
