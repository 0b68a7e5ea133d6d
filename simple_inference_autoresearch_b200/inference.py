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
    ap.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--prompt", help="prompt text (needs tokenizer.json in the model folder)")
    ap.add_argument("--prompt-ids", help="prompt as comma- or space-separated token ids")
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at the model's stop tokens")
    ap.add_argument("--no-cuda-graph", action="store_true")
    args = ap.parse_args(argv)

    import simple_inference_autoresearch_b200 as siar

    model_dir = Path(args.model)
    tok = _tokenizer(model_dir)
    loaded = siar.load_model(model_dir, device="cuda", dtype=args.dtype)
    if args.prompt_ids:
        ids = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
    elif args.prompt is not None:
        if tok is None:
            ap.error("--prompt needs tokenizer.json in the model folder and the 'tokenizers' package; "
                     "use --prompt-ids")
        ids = tok.encode(args.prompt, add_special_tokens=False).ids
        ids = [loaded.config.bos_token_id] + ids          # add_bos=True, as tokenizer.py:74-85
    else:
        ap.error("one of --prompt / --prompt-ids is required")
    engine = siar.build_engine(loaded, max_batch=1, max_seq_len=len(ids) + args.max_new_tokens,
                               use_cuda_graph=not args.no_cuda_graph)

    def on_token(t: int) -> None:
        print(tok.decode([t]) if tok is not None else f"{t} ", end="", flush=True)

    out, stats = siar.generate_with_stats(ids, engine, max_new_tokens=args.max_new_tokens,
                                          temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                                          on_token=on_token, seed=args.seed, ignore_eos=args.ignore_eos)
    if out:
        print()
    width = max(len(k) for k in stats)
    print("-" * (width + 16))
    for k, v in stats.items():
        print(f"{k:<{width}} : {v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
