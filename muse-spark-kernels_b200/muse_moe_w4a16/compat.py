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

The prefill layer calls
    ex = _moe_forward(st, p, lid, pos, cnt, T, zb=..., cit=cit)      # y rows + row map, or the combined output via cit
    moe_combine(y, rrow, lid, topw, g_post_expert_norm, moe)            # unless combined in the kernel's tail
(muse_prefill_layer/py/04_moe_forward.py:6-52, py/06_kernel_fn.py:100-118) with the un-normed pooler
output p, local ids and the routing weights. `PrefillMoe.moe_forward` takes that call's arguments and
returns the combined output: pre-expert norm, both GEMMs, post-expert norm and the weighted sum are
one kernel_fn call on a state prepared with pre_norm_w / post_norm_w.
"""
import torch

from . import attrs, kernel_fn, workspace_views


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


class PrefillMoe:
    """Stand-in for the prefill layer's expert step. state: prepare(weights with pre_norm_w =
    g_pre_expert_norm and post_norm_w = g_post_expert_norm, local_start=0, n_experts=local experts,
    top_k=8, max_tokens=largest T)."""

    def __init__(self, state):
        self.state = state

    def __deepcopy__(self, memo):
        return self

    def moe_forward(self, p, lid, pos, cnt, T, topw, out=None, order=None, zb=None):
        """p bf16 [T, H] (pooler output, not normed), lid int32 [T, k] local ids (-1 = another rank's
        expert), topw fp32 [T, k]. pos / cnt / order / zb are the reference's per-expert positions,
        counts, tile order and zeroed counters: this library derives its own (deterministic) tables
        from lid, so they are accepted and not read. Returns dict(out=bf16 [T, H] combined output,
        rrow=int32 [T, k] row of each route in the sorted order or -1): `out` is what the reference's
        cit path leaves in cit["out"], rrow what its gather writes."""
        if int(T) != p.shape[0] or tuple(lid.shape) != tuple(topw.shape):
            raise RuntimeError("moe_forward: T, lid and topw do not agree")
        res = kernel_fn({"hidden_states": p, "topk_ids": lid, "topk_weights": topw}, self.state, out=out)
        return {"out": res, "rrow": _RowMap(self.state, int(T))}

    def moe_combine(self, y, rrow, lid, topw, g_post, out):
        """The combine already ran inside moe_forward; kept so that the call site stays as it is."""
        return None


class _RowMap:
    """rrow on demand (it lives in the workspace until the next call): tensor() copies it out."""

    def __init__(self, state, T):
        self.state, self.T = state, T

    def tensor(self):
        return workspace_views(self.state, self.T)["inv"].view(self.T, self.state["cfg"].top_k)
