"""Generates tests/golden/reference_vectors.npz from the reference's own importable Python.

Run in the build container only (it reads the reference checkout; the GPU box has none):
    python tests/golden/make_golden.py [/path/to/reference]
The reference module is assembled in memory with the reference's build.assemble() and
executed on CPU; nothing of it is written into this repository except the numeric vectors:
  nib_codes / nib_rows / nib_out   `_split_nibbles(codes, rows)`: nibble order (low nibble = even k)
  e4m3_lut                         the 256-entry scale table expression of prepare():
                                   e4m3 byte -> bf16x2(value * 2^64) packed in an int32
  gen{bs}_ids / gen{bs}_w          `_gen_input(bs, seed=0, cpu)`: harness-style top-8 ids
                                   (busiest-rank relabel) and normalised weights
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path of the reference checkout>")
REF = sys.argv[1]
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")


def load_reference_module():
    spec = importlib.util.spec_from_file_location("_ref_build", os.path.join(REF, "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    src = b.assemble("muse_moe_w4a16")
    mod = types.ModuleType("ref_muse_moe_w4a16")
    exec(compile(src, "ref_muse_moe_w4a16.py", "exec"), mod.__dict__)
    return mod


def main():
    ref = load_reference_module()
    g = torch.Generator().manual_seed(1234)
    codes = torch.randint(0, 256, (6, 32), generator=g, dtype=torch.uint8)
    rows = torch.tensor([3, 0, 5, 1])
    nib, _ = ref._split_nibbles(codes, rows)
    # the table expression of prepare() (muse_moe_w4a16/py/02_prepare.py:31-33), evaluated as written there
    lut = (torch.arange(256, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn).float()
           * 2.0 ** 64).to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    lut = (lut | (lut << 16)).to(torch.int32)
    out = {"nib_codes": codes.numpy(), "nib_rows": rows.numpy(), "nib_out": nib.numpy(), "e4m3_lut": lut.numpy()}
    for bs in (4, 33):
        d = ref._gen_input(bs, 0, torch.device("cpu"))
        out[f"gen{bs}_ids"] = d["topk_ids"].numpy()
        out[f"gen{bs}_w"] = d["topk_weights"].numpy()
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
