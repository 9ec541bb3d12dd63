"""Compile the reference's own kernels for sm_100a into oracle/_ref/ (git-ignored).

The reference ships its GPU kernels as PTX text inside Rust string literals
(crates/oxide-infer-kernels/src/batched_attn.rs).  This recipe reads each
``pub const NAME: &str = r#"..."#;`` literal where it lies in the reference
checkout, hands the text to ``ptxas -arch=sm_100a`` (the same translation the
driver's JIT performs when the reference loads the string) and keeps only the
resulting machine-code image ``oracle/_ref/NAME.cubin``.  No reference source is
written into the repository.  The cubins are what tests and the benchmark's
reference arm execute on the GPU; they are TEST INFRASTRUCTURE, never part of
the product library.

Usage: python oracle/build_ref.py [--reference /path/to/reference]
The checkout is found through --reference, else the environment variable OXIDE_INFER_REFERENCE,
else a directory named "reference" beside this repository.  Exits 0 and prints "reference not
present" when none of them holds the file.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REL = "crates/oxide-infer-kernels/src/batched_attn.rs"

# PTX constants on (or used to check) the pointer-table path.
WANTED = [
    "BATCHED_QK_RMSNORM_PTX", "BATCHED_ROPE_PTX", "BATCHED_KV_COPY_PTX",
    "BATCHED_GQA_ATTENTION_ONLINE_PTX", "BATCHED_GQA_ATTENTION_SPLIT_PTX",
    "BATCHED_GQA_ATTENTION_SPLIT4_PTX", "BATCHED_SIGMOID_GATE_PTX", "BATCHED_CONV_PTR_PTX",
    "CONV_STATE_PREFILL_PTX", "BATCHED_ATTN_PACK_Q_PTX", "BATCHED_ATTN_SOFTMAX_MASK_PTX",
    "BATCHED_ATTN_GATE_SCATTER_PTX",
    # the two other table-driven kernels of the same file (sampling side of a decode step)
    "BATCHED_EMBED_LOOKUP_PTX", "BATCHED_ARGMAX_DIRECT_PTX",
]


def default_reference() -> str:
    """OXIDE_INFER_REFERENCE, else <parent of the repository>/reference."""
    return os.environ.get("OXIDE_INFER_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference: str | None = None, verbose: bool = True) -> int:
    src = os.path.join(reference or default_reference(), REL)
    if not os.path.exists(src):
        if verbose:
            print("reference not present; oracle/_ref left as is")
        return 0
    text = open(src, encoding="utf-8").read()
    lits = dict(re.findall(r'pub const (\w+): &str = r#"(.*?)"#;', text, flags=re.S))
    os.makedirs(OUT, exist_ok=True)
    n = 0
    for name in WANTED:
        if name not in lits:
            raise SystemExit(f"{name} not found in {src}")
        with tempfile.NamedTemporaryFile("w", suffix=".ptx", dir=tempfile.gettempdir(),
                                         delete=True) as f:
            f.write(lits[name])
            f.flush()
            out = os.path.join(OUT, name + ".cubin")
            subprocess.run(["ptxas", "-arch=sm_100a", "-o", out, f.name], check=True)
        n += 1
    if verbose:
        print(f"built {n} cubins into {OUT}")
    return n


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    a = ap.parse_args()
    build(a.reference)
    sys.exit(0)
