"""``python inference.py --model DIR --prompt-ids ... `` — see simple_inference_autoresearch_b200/inference.py."""
import sys

from simple_inference_autoresearch_b200.inference import main

if __name__ == "__main__":
    sys.exit(main())
