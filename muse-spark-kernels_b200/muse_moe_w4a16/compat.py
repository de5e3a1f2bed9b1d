"""Stand-in for the extension object of the reference module, for its layer callers.

The decode layer gets an object from `_moe(T, state)` and calls
    ext.okc_set_pdl(1 if pdl else 0)
    ext.okc_run(state["ma_w"], state["ma_scratch"], x, lids, wts, out, 0, 32, state["nsm"])
(muse_decode_layer/py/06_kernel_fn.py:140-149; interface muse_moe_w4a16/py/00_moe_w4a16.py:208-214,
muse_moe_w4a16/cuda/moe.cu:2787-2881), with *local* expert ids and -1 for another GPU's expert,
in chunks of at most 384 tokens. `OkcExt` has the same three methods over a state prepared by
this package, so that call site runs unchanged:

    state["okc"] = OkcExt(prepare(weights, local_start=0, n_experts=32, top_k=8, max_tokens=384))
    ext = state["okc"]          # what _moe(T, state) returns
"""
import torch

from . import attrs, kernel_fn


class OkcExt:
    def __init__(self, state):
        self.state = state

    def __deepcopy__(self, memo):            # the harness deep-copies states; handles are shared
        return self

    def okc_set_pdl(self, on):
        """The reference's process-wide switch (muse_moe_w4a16/cuda/moe.cu:2348,2565) as a field of this
        state's configuration: with 0 the launches of a step are plain stream-ordered launches, with 1
        they are chained with programmatic dependent launch (the default)."""
        self.state["cfg"].no_pdl = 0 if on else 1
        return None

    def okc_attrs(self):
        """[registers, local bytes, static shared bytes] of the gate/up and the down GEMM kernel
        (narrow token tile), the shape of the reference's six numbers."""
        a, b = attrs(2, 16), attrs(3, 16)
        return [a[0], a[3], a[1], b[0], b[3], b[1]]

    def okc_run(self, w, scratch, x, ids, tw, out, lo, nloc, grid):
        """`w` and `scratch` are the reference's tensor lists; the prepared state owns their
        counterparts, so they are not read. `lo` / `nloc` must be the prepared local range and `grid`
        the persistent grid the state was prepared for (num_ctas, 148 by default): a call that asks for
        another one is refused rather than silently run on a different grid."""
        st = self.state
        if int(lo) != st["lo"] or int(nloc) != st["cnt"]:
            raise RuntimeError("okc_run: local range differs from the prepared state")
        want = st["cfg"].num_ctas or 148
        if int(grid) != want:
            raise RuntimeError(f"okc_run: grid {int(grid)} differs from the prepared state's {want}")
        kernel_fn({"hidden_states": x, "topk_ids": ids, "topk_weights": tw}, st, out=out)
        return None
