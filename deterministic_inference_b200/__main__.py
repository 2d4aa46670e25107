"""Command line: ``python -m deterministic_inference_b200 <command>``.

The reference's only command lines are its server and its kernel build
(sid/server.py:188-208, sid/kernels/jit.py:66-67); option names that exist there
keep their names here (``--model``, ``--kv-pool-tokens``).

  generate   run prompts (token ids) to completion and print the generated ids
  random     write a model folder with random weights from a preset and a seed
  build      compile every CUDA library for sm_100a
  replay     trace replay (the program bin/trace_run: steps on standard input, logits to disk)
  bench      the benchmark (the program bench.py at the repository root)
"""

from __future__ import annotations

import argparse
import json
import sys


def _cmd_generate(a) -> int:
    import torch

    from .config import EngineConfig, SamplingParams, preset
    from .engine import Engine

    if (a.model is None) == (a.preset is None):
        print("give exactly one of --model DIR or --preset NAME", file=sys.stderr)
        return 2
    kw = dict(dtype=a.dtype, kv_pool_tokens=a.kv_pool_tokens, page_size=a.page_size,
              max_reqs=a.max_reqs, max_seq_len=a.max_seq_len,
              max_prefill_tokens=a.max_prefill_tokens, max_decode_batch=a.max_decode_batch,
              cuda_graphs=not a.no_cuda_graphs, async_scheduling=not a.no_async_scheduling,
              device=a.device)
    if a.model is not None:
        cfg = EngineConfig(model_path=a.model, **kw)
    else:
        cfg = EngineConfig(model_config=preset(a.preset), random_seed=a.random_seed, **kw)
    engine = Engine(cfg)
    prompts = []
    if a.prompt_ids:
        prompts += [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    if a.prompt_lens:
        g = torch.Generator().manual_seed(a.prompt_seed)
        for n in a.prompt_lens.split(","):
            prompts.append(torch.randint(0, engine.vocab_size, (int(n),), generator=g).tolist())
    if a.prompt:
        prompts += a.prompt
    if not prompts:
        print("no prompt: give --prompt-ids, --prompt-lens or --prompt", file=sys.stderr)
        return 2
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                        max_new_tokens=a.max_new_tokens, seed=a.seed, ignore_eos=a.ignore_eos)
    for out in engine.generate(prompts, sp):
        print(json.dumps({"rid": out.rid, "prompt_len": len(out.prompt_ids),
                          "token_ids": out.token_ids, "text": out.text,
                          "finish_reason": out.finish_reason}))
    return 0


def _cmd_random(a) -> int:
    from .config import preset
    from .weights import write_random_model

    d = write_random_model(preset(a.preset), a.seed, a.out)
    print(d)
    return 0


def _cmd_build(a) -> int:
    from .kernels import build

    for name, path in sorted(build.compile_all().items()):
        print(f"{name}: {path}")
    return 0


def _run_script(path, args) -> int:
    import runpy
    from pathlib import Path

    script = Path(__file__).resolve().parent.parent / path
    if not script.exists():
        print(f"{script} is not there (this command needs the repository checkout)", file=sys.stderr)
        return 2
    old = sys.argv
    sys.argv = [str(script)] + list(args)
    try:
        runpy.run_path(str(script), run_name="__main__")
    except SystemExit as e:
        return int(e.code or 0)
    finally:
        sys.argv = old
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        return _run_script("bin/trace_run", argv[1:])
    if argv and argv[0] == "bench":
        return _run_script("bench.py", argv[1:])
    ap = argparse.ArgumentParser(prog="python -m deterministic_inference_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    g = sub.add_parser("generate", help="generate from token-id prompts")
    g.add_argument("--model", help="folder with config.json and *.safetensors")
    g.add_argument("--preset", help="a named shape with random weights instead of a folder")
    g.add_argument("--random-seed", type=int, default=0)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", help='"1,2,3"; may be repeated')
    g.add_argument("--prompt-lens", help='"5,17,33": random prompts of these lengths')
    g.add_argument("--prompt-seed", type=int, default=1)
    g.add_argument("--prompt", action="append", help="text (needs a tokenizer in the folder)")
    g.add_argument("--max-new-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--kv-pool-tokens", type=int, default=256 * 1024)
    g.add_argument("--page-size", type=int, default=16)
    g.add_argument("--max-reqs", type=int, default=256)
    g.add_argument("--max-seq-len", type=int, default=32768)
    g.add_argument("--max-prefill-tokens", type=int, default=8192)
    g.add_argument("--max-decode-batch", type=int, default=256)
    g.add_argument("--no-cuda-graphs", action="store_true")
    g.add_argument("--no-async-scheduling", action="store_true")
    g.add_argument("--device", default="cuda")
    g.set_defaults(fn=_cmd_generate)

    r = sub.add_parser("random", help="write a random-weights model folder")
    r.add_argument("--preset", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.set_defaults(fn=_cmd_random)

    b = sub.add_parser("build", help="compile the CUDA libraries")
    b.set_defaults(fn=_cmd_build)

    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
