"""Generates tests/golden/reference_vectors.npz from the reference's own Python, run on the CPU.

Run in the build container only (it reads the reference checkout; the GPU box has none):
    python tests/golden/make_golden.py /path/to/reference
Nothing of the reference is written into this repository except the numeric vectors. Two ways of
running reference code are used:
  * the module `muse_moe_w4a16` is assembled in memory with the reference's build.assemble() and
    executed on the CPU (packers, input generator);
  * Triton kernels of `muse_decode_layer` (plain @triton.jit functions) are cut out of the reference
    file by name into a temporary module and run with Triton's CPU interpreter (TRITON_INTERPRET=1).
    The two programmatic-dependent-launch helpers they call have no numeric effect and are replaced
    by empty functions for the interpreter.
Vectors:
  nib_codes / nib_rows / nib_out   `_split_nibbles(codes, rows)`: nibble order (low nibble = even k)
  e4m3_lut                         the 256-entry scale table of prepare(), computed by executing the
                                   statements of muse_moe_w4a16/py/02_prepare.py that build `lut`
  gen{bs}_ids / gen{bs}_w          `_gen_input(bs, seed=0, cpu)`: harness-style top-8 ids and weights
  rs_*                             `_route_split` (muse_decode_layer/py/04_triton_kernels.py:565-609):
                                   inputs pooled / logits / bias / gpre / local_start, outputs ids, lids,
                                   weights and the pre-expert-normed rows; the logits hold exact ties
  lk_ids / lk_w                    `_link_route` with the packed 64-bit key (sort form,
                                   muse_decode_layer/py/07_link_chain.py:101-112) on the same inputs
  pn_*                             `_pexp_norm_sum` (04_triton_kernels.py:616-632): per-route rows,
                                   post-norm weight, routing weights, local ids (-1 = skipped) -> out
"""
import importlib.util
import os
import re
import sys
import tempfile
import types

os.environ["TRITON_INTERPRET"] = "1"   # before triton is imported

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


def reference_lut():
    """Executes the reference's own statements that build the E4M3 table (the two assignments to
    `lut` inside prepare()), with dev = cpu."""
    text = open(os.path.join(REF, "muse_moe_w4a16", "py", "02_prepare.py")).read()
    stmts = re.findall(r"^    (lut = .*?)(?=^    \S)", text, flags=re.S | re.M)
    assert len(stmts) == 2, "expected the two `lut = ...` statements of prepare()"
    ns = {"torch": torch, "dev": torch.device("cpu")}
    for s in stmts:
        exec("\n".join(line[4:] if line.startswith("    ") else line for line in s.splitlines()), ns)
    return ns["lut"]


def triton_kernels(rel_path, names, stubs=()):
    """Cuts the named @triton.jit functions out of a reference file into a temporary module."""
    text = open(os.path.join(REF, rel_path)).read()
    parts = ["import triton\nimport triton.language as tl\n"]
    for s in stubs:
        parts.append(f"@triton.jit\ndef {s}():\n    pass\n")
    for n in names:
        m = re.search(r"^@triton\.jit\ndef %s\(.*?(?=^\S)" % re.escape(n), text, flags=re.S | re.M)
        assert m, n
        parts.append(m.group(0))
    d = tempfile.mkdtemp()
    path = os.path.join(d, "ref_triton_" + names[0].strip("_") + ".py")
    with open(path, "w") as f:
        f.write("\n".join(parts))
    spec = importlib.util.spec_from_file_location(os.path.basename(path)[:-3], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = load_reference_module()
    g = torch.Generator().manual_seed(1234)
    codes = torch.randint(0, 256, (6, 32), generator=g, dtype=torch.uint8)
    rows = torch.tensor([3, 0, 5, 1])
    nib, _ = ref._split_nibbles(codes, rows)
    out = {"nib_codes": codes.numpy(), "nib_rows": rows.numpy(), "nib_out": nib.numpy(),
           "e4m3_lut": reference_lut().numpy()}
    for bs in (4, 33):
        d = ref._gen_input(bs, 0, torch.device("cpu"))
        out[f"gen{bs}_ids"] = d["topk_ids"].numpy()
        out[f"gen{bs}_w"] = d["topk_weights"].numpy()

    # ---- routing + pre-expert norm: _route_split, and _link_route's packed-key form
    T = 6
    g = torch.Generator().manual_seed(77)
    pooled = (torch.randn((T, 4096), generator=g) * 1.7).to(torch.bfloat16)
    logits = torch.randn((T, 256), generator=g) * 2.0
    bias = torch.randn((256,), generator=g) * 0.1
    # exact ties: experts 8..15 repeat the logits and the bias of experts 200..207 (the lower index must
    # win), and token 1 has one value everywhere (the top-8 are then experts 0..7 in the order of the bias)
    logits[:, 8:16] = logits[:, 200:208]
    bias[8:16] = bias[200:208]
    logits[1, :] = 0.25
    gpre = (torch.randn((4096,), generator=g) * 0.1).to(torch.bfloat16)
    ls = torch.tensor([64], dtype=torch.int32)
    k1 = triton_kernels("muse_decode_layer/py/04_triton_kernels.py", ["_route_split", "_pexp_norm_sum"])
    ids = torch.zeros((T, 8), dtype=torch.int32)
    lids = torch.zeros((T, 8), dtype=torch.int32)
    wts = torch.zeros((T, 8), dtype=torch.float32)
    xout = torch.zeros((T, 4096), dtype=torch.bfloat16)
    k1._route_split[(T,)](pooled, logits, bias, gpre, ids, wts, xout, ls, lids, PERMUTED=False)
    out.update({"rs_pooled": pooled.view(torch.int16).numpy(), "rs_logits": logits.numpy(), "rs_bias": bias.numpy(),
                "rs_gpre": gpre.view(torch.int16).numpy(), "rs_local_start": ls.numpy(), "rs_ids": ids.numpy(),
                "rs_lids": lids.numpy(), "rs_w": wts.numpy(), "rs_x": xout.view(torch.int16).numpy()})
    try:
        k2 = triton_kernels("muse_decode_layer/py/07_link_chain.py", ["_link_route"], stubs=("_gdc_launch", "_gdc_wait"))
        ids2 = torch.zeros((T, 8), dtype=torch.int32)
        lids2 = torch.zeros((T, 8), dtype=torch.int32)
        wts2 = torch.zeros((T, 8), dtype=torch.float32)
        x2 = torch.zeros((T, 4096), dtype=torch.bfloat16)
        k2._link_route[(T, 2)](pooled, logits, logits, bias, gpre, ids2, wts2, x2, ls, lids2, SPLIT=True, EARLY=False,
                               PACKED=2)
        out.update({"lk_ids": ids2.numpy(), "lk_w": wts2.numpy()})
    except Exception as exc:  # the interpreter may lack tl.sort / tl.gather; the argmax form above still pins the rule
        print("packed-key form not generated:", type(exc).__name__, exc)

    # ---- post-expert norm + weighted sum: _pexp_norm_sum
    Tn, K, H = 5, 8, 512
    g = torch.Generator().manual_seed(78)
    y = (torch.randn((Tn * K, H), generator=g) * 3.0).to(torch.bfloat16)
    pw = (torch.randn((H,), generator=g) * 0.1).to(torch.bfloat16)
    sw = torch.rand((Tn, K), generator=g)
    pid = torch.randint(-1, 32, (Tn, K), generator=g, dtype=torch.int32)
    pid[2] = -1                      # a token without any local route
    pout = torch.zeros((Tn, H), dtype=torch.bfloat16)
    k1._pexp_norm_sum[(Tn,)](y, pw, sw, pout, pid, TOPK=K, H=H, eps=1e-8, BLOCK_H=512)
    out.update({"pn_y": y.view(torch.int16).numpy(), "pn_w": pw.view(torch.int16).numpy(), "pn_s": sw.numpy(),
                "pn_ids": pid.numpy(), "pn_out": pout.view(torch.int16).numpy()})
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
