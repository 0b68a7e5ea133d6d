"""Runs the reference project's own ``sampling.sample`` on the CPU for a few rows of logits and
stores the probabilities it draws from, so that ``tests/plain_llama.kept_probabilities`` can be
compared with them without the reference present.

    USE_FUSED_SAMPLE=false python tests/golden/make_sampler_golden.py /path/to/reference

The reference draws with ``torch.multinomial`` (sampling.py:224,236); this script swaps that one
torch function for a recorder while ``sample`` runs, which leaves the reference's code as it is and
yields the exact categorical distribution behind every draw: over the k candidates of the top-k
path (sampling.py:203-225, scattered back to token ids here) or over the whole vocabulary
(sampling.py:229-236).  The rows hold no equal logits: where logits tie at the k-th place or at the
nucleus edge the reference's result depends on the order its sort happens to give them
(sampling.py:200-202), and the plain implementation keeps tied tokens together instead.
"""

import json
import os
import sys
from pathlib import Path

os.environ.setdefault("USE_FUSED_SAMPLE", "false")
os.environ.setdefault("USE_TRITON", "false")

import torch  # noqa: E402

HERE = Path(__file__).resolve().parent

CASES = [  # (temperature, top_k, top_p)
    (1.0, 0, 1.0), (0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 50, 0.9), (1.3, 0, 0.6), (1.0, 1, 1.0), (0.5, 40, 0.0),
    (1.0, 0, 0.0), (1.0, 100000, 0.95), (2.0, 7, 0.5), (0.3, 0, 0.99),
]


def main(ref_path: str) -> None:
    sys.path.insert(0, ref_path)
    import sampling

    g = torch.Generator().manual_seed(77)
    rows = torch.randn(4, 300, generator=g) * 2.0
    rows[1] *= 3.0                       # a peaked row
    rows[2] *= 0.05                      # a flat row
    assert all(r.unique().numel() == r.numel() for r in rows)
    out = {"logits": rows.contiguous()}
    seen = {}
    real = torch.multinomial

    def recorder(probs, num_samples=1, **kw):
        seen["probs"] = probs.detach().clone()
        return real(probs, num_samples, **kw)

    for ci, (t, k, p) in enumerate(CASES):
        full = torch.zeros_like(rows, dtype=torch.float64)
        for ri in range(rows.shape[0]):
            torch.multinomial = recorder
            try:
                sampling.sample(rows[ri:ri + 1], temperature=t, top_k=k, top_p=p)
            finally:
                torch.multinomial = real
            probs = seen["probs"][0].double()
            if 0 < k < rows.shape[1]:        # the candidates of the top-k path, in descending order of logit
                idx = torch.topk(rows[ri], k, largest=True, sorted=True).indices
                full[ri, idx] = probs
            else:
                full[ri] = probs
        out[f"probs{ci}"] = full.float().contiguous()
    from safetensors.torch import save_file
    save_file(out, str(HERE / "sampler.safetensors"), metadata={"cases": json.dumps(CASES)})
    print("saved", sum(v.numel() for v in out.values()) * 4 // 1024, "KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_sampler_golden.py /path/to/reference")
    main(sys.argv[1])
