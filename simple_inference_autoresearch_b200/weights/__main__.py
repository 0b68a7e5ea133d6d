"""``python -m simple_inference_autoresearch_b200.weights --config FILE --out DIR --seed N``: writes a
model folder (config.json, model.safetensors) with seeded random weights, see ``random_init``."""
import sys

from .random_init import main

if __name__ == "__main__":
    sys.exit(main())
