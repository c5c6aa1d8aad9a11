"""numpy restatement of MoEFeedForward.forward at world size 1
(polkadot21/fastmoe, src/fastmoe/models/tiny_model.py:411-420), fp32.

TEST INFRASTRUCTURE — see oracle/__init__.py.
"""

from __future__ import annotations

import math

import numpy as np

from .routing import build_index, topk_softmax

_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu(x: np.ndarray) -> np.ndarray:
    """nn.GELU() default (erf form), tiny_model.py:72."""
    x64 = x.astype(np.float64)
    return (0.5 * x64 * (1.0 + _erf(x64 / math.sqrt(2.0)))).astype(np.float32)


def moe_layer_forward(x, router_w, w1, w2, K):
    """x [T, D]; router_w [E, D]; w1[e] [ff, D]; w2[e] [D, ff] (nn.Linear layout, no bias).

    gate_and_sort (:79-164) -> compute_experts (:282-294) -> unpermute (:396-409).
    Returns (out [T, D], intermediates dict).
    """
    x = np.asarray(x, dtype=np.float32)
    T, D = x.shape
    E = router_w.shape[0]
    logits = x @ router_w.T.astype(np.float32)
    idx, w = topk_softmax(logits, K)
    ix = build_index(idx, w, E)
    permuted = x[ix["reverse_map"]]
    outs = []
    for e in range(E):
        lo, n = int(ix["offsets"][e]), int(ix["counts"][e])
        chunk = permuted[lo : lo + n]
        outs.append(gelu(chunk @ w1[e].T) @ w2[e].T if n else np.zeros((0, D), np.float32))
    out = np.zeros((T, D), np.float32)
    rows = np.concatenate(outs, axis=0)
    # out.index_add_(0, reverse_map, rows * w) in slot order (ops.py:373-384 with one tensor)
    np.add.at(out, ix["reverse_map"], rows * ix["sorted_w"][:, None])
    return out, {"logits": logits, "topk_idx": idx, "topk_w": w, "permuted": permuted, "rows": rows, **ix}
