"""Command line in the manner of the reference's ``inference.py`` (inference.py:19-53):

    python inference.py --model DIR (--prompt TEXT | --prompt-ids 1,2,3) \
        [--max-new-tokens 128] [--temperature 0.7] [--top-k 50] [--top-p 0.9]

``--model``, ``--prompt``, ``--max-new-tokens``, ``--temperature``, ``--top-k`` and ``--top-p`` keep
the reference's names, meanings and defaults; the cache is sized for the prompt plus the new
tokens, batch 1, tokens are streamed as they come and the reference's metrics are printed
(utilities.py:74-92).  Differences: ``--model`` is a local folder (config.json +
safetensors; nothing is downloaded), and since the library works on token ids, ``--prompt`` text
needs a ``tokenizer.json`` in that folder (read with the ``tokenizers`` package); ``--prompt-ids``
always works.  ``--dtype float32`` runs the true 32-bit path.

Beyond the reference: ``--model NAME --random-weights`` takes one of the configurations shipped
with the library (``tiny-a``, ``tiny-b``, ``llama-3.2-1b``, ``llama-3.2-3b``, ``llama-3.1-8b``) or
added with ``config.register_preset``, of whatever registered architecture its config.json names, with
seeded random weights made on the GPU (``--seed``; ``--norm-init`` overrides the configuration's rule for norm weights); ``--prompt-len N`` feeds N seeded random
token ids; ``--batch N`` generates for N prompts at once (``--prompt-len`` draws N different
ones, their lengths spread between N/2 and N tokens; a given prompt is repeated) and prints the token
lists instead of streaming; ``--stop-id ID`` (repeatable) adds stop tokens to the model's own.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path


def _tokenizer(model_dir: Path):
    path = model_dir / "tokenizer.json"
    if not path.exists():
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(str(path))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True,
                    help="model folder (config.json + model.safetensors), or with --random-weights the name of a "
                         "shipped configuration")
    ap.add_argument("--random-weights", action="store_true",
                    help="seeded random weights for the configuration --model names (a shipped name or a folder's config.json)")
    ap.add_argument("--norm-init", choices=["ones", "ones_plus_normal"],
                    help="with --random-weights: norm weights 1 or 1 + N(0, initializer_range) (default: the configuration's)")
    ap.add_argument("--prompt", help="prompt text (needs tokenizer.json in the model folder)")
    ap.add_argument("--prompt-ids", help="prompt as comma- or space-separated token ids")
    ap.add_argument("--prompt-len", type=int, help="a prompt of this many seeded random token ids")
    ap.add_argument("--batch", type=int, default=1, help="number of prompts generated for at once")
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stop-id", type=int, action="append", default=[], help="a further stop token id (repeatable)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at the model's stop tokens")
    ap.add_argument("--no-cuda-graph", action="store_true")
    args = ap.parse_args(argv)
    if args.batch < 1:
        ap.error("--batch must be at least 1")

    import simple_inference_autoresearch_b200 as siar

    model_dir = Path(args.model)
    tok = _tokenizer(model_dir) if model_dir.is_dir() else None
    if args.random_weights:
        from . import registry
        from .config import preset_path
        try:
            config_file = model_dir / "config.json" if model_dir.is_dir() else preset_path(args.model)
        except FileNotFoundError as e:
            ap.error(str(e))
        _arch, config = registry.resolve_path(config_file)      # the class config.json's architecture names
        options = {"norm_weight_init": args.norm_init} if args.norm_init else {}
        loaded = siar.init_random(siar.build_model(config, args.dtype, "cuda", **options), args.seed)
    elif not model_dir.is_dir():
        ap.error(f"--model {args.model}: no such folder (a shipped configuration needs --random-weights)")
    else:
        loaded = siar.load_model(model_dir, device="cuda", dtype=args.dtype)
    if args.prompt_ids:
        prompts = [[int(t) for t in args.prompt_ids.replace(",", " ").split()]] * args.batch
    elif args.prompt is not None:
        if tok is None:
            ap.error("--prompt needs tokenizer.json in the model folder and the 'tokenizers' package; "
                     "use --prompt-ids")
        ids = tok.encode(args.prompt, add_special_tokens=False).ids
        prompts = [[loaded.config.bos_token_id] + ids] * args.batch   # add_bos=True, as tokenizer.py:74-85
    elif args.prompt_len:
        import torch
        g = torch.Generator().manual_seed(args.seed)
        n = args.prompt_len
        lengths = [n] if args.batch == 1 else [max(1, n - (n // 2) * j // (args.batch - 1)) for j in range(args.batch)]
        prompts = [torch.randint(0, loaded.config.vocab_size, (m,), generator=g).tolist() for m in lengths]
    else:
        ap.error("one of --prompt / --prompt-ids / --prompt-len is required")
    engine = siar.build_engine(loaded, max_batch=args.batch,
                               max_seq_len=max(len(p) for p in prompts) + args.max_new_tokens,
                               use_cuda_graph=not args.no_cuda_graph)
    if args.batch > 1:
        params = siar.SamplingParams(args.temperature, args.top_k, args.top_p, args.seed)
        outs, stats = engine.generate(prompts, params, args.max_new_tokens, stop_token_ids=args.stop_id or None,
                                      ignore_eos=args.ignore_eos, return_stats=True)
        for j, (p, o) in enumerate(zip(prompts, outs)):
            print(f"[{j}] {len(p)} prompt tokens -> {' '.join(str(t) for t in o)}")
        _print_stats(stats)
        return 0
    ids = prompts[0]

    def on_token(t: int) -> None:
        print(tok.decode([t]) if tok is not None else f"{t} ", end="", flush=True)

    out, stats = siar.generate_with_stats(ids, engine, max_new_tokens=args.max_new_tokens,
                                          temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                                          on_token=on_token, seed=args.seed, stop_token_ids=args.stop_id or None,
                                          ignore_eos=args.ignore_eos)
    if out:
        print()
    _print_stats(stats)
    return 0


def _print_stats(stats: dict) -> None:
    width = max(len(k) for k in stats)
    print("-" * (width + 16))
    for k, v in stats.items():
        print(f"{k:<{width}} : {v}")


if __name__ == "__main__":
    sys.exit(main())
