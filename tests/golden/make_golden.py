"""Writes tests/golden/plain_tiny_logits.npz: logits of the plain implementation on two tiny random
models.  integrallis/models' own model code cannot be compiled or imported here (a Java 25 library
with an external numeric core; no JVM or build tool is installed), so these files do not come from
it: they pin the plain implementation, which rests on the reference's formulas, against accidental
change.  Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def compute():
    from plain import plain_llama
    from tiny import TINY_A, TINY_B, make_folder, random_tokens

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, raw in (("A", TINY_A), ("B", TINY_B)):
            folder = make_folder(raw, 42, os.path.join(tmp, name))
            config, weights = plain_llama.read_model_folder(folder)
            tokens = random_tokens(raw["vocab_size"], 12, 42)
            logits = plain_llama.forward(config, weights, tokens)
            out[name] = logits[[0, 5, 11]][:, :16].numpy()
    return out


if __name__ == "__main__":
    np.savez(os.path.join(HERE, "plain_tiny_logits.npz"), **compute())
    print("wrote plain_tiny_logits.npz")
