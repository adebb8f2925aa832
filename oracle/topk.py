"""CPU restatement of the reference's top-k position selection (test infrastructure only).

Follows flash_sparse_attn/utils/mask.py:20-44: ``torch.topk(attention_bias, window_size, dim=-1,
largest=True, sorted=False).indices`` followed by ``torch.sort`` of the indices. torch leaves the choice
among EQUAL scores at the threshold unspecified; this restatement (and the CUDA kernel) take the lowest
positions, so parity with the reference is pinned for rows without ties at the threshold
(tests/golden/topk.npz) and stated, not pinned, for rows with ties.
"""

import numpy as np


def order_keys(x: np.ndarray) -> np.ndarray:
    """Monotone map float32 -> uint32 (larger value, larger key; NaN above +inf), as the kernel uses."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000)).astype(np.uint32)


def topk_indices(scores: np.ndarray, k: int) -> np.ndarray:
    """scores [..., n] -> int64 [..., k]: ascending positions of the k largest entries (ties: lowest positions)."""
    x = np.asarray(scores, dtype=np.float32)
    flat = x.reshape(-1, x.shape[-1])
    out = np.empty((flat.shape[0], k), dtype=np.int64)
    for r in range(flat.shape[0]):
        keys = order_keys(flat[r]).astype(np.int64)
        # stable sort by descending key keeps lower positions first among equals
        order = np.argsort(-keys, kind="stable")[:k]
        out[r] = np.sort(order)
    return out.reshape(*x.shape[:-1], k)
