"""Test helpers with the reference's names (gemm/BF16/utils.py:5-44)."""

import random

import torch


def gmm(a, b, batch_sizes, trans_b=False):
    """Per-group torch product -- the reference's correctness baseline."""
    pieces, row = [], 0
    for g, rows in enumerate(batch_sizes.tolist()):
        w = b[g].t() if trans_b else b[g]
        pieces.append(a[row:row + rows] @ w)
        row += rows
    return torch.cat(pieces)


def allclose(x, y, pct=2.0):
    close = torch.isclose(x, y, rtol=1e-5)
    bad = 100.0 * (close.numel() - int(close.sum())) / close.numel()
    if bad > pct:
        print(f"{bad:.2f}% of values not close.")
        return False
    return True


def generate_random_list(length, total_sum):
    """`length` non-negative ints that add up to `total_sum` (random split)."""
    avg = total_sum // length
    raw = [random.randint(0, 2 * int(avg)) for _ in range(length)]
    scale = total_sum / max(sum(raw), 1)
    out = [int(v * scale) for v in raw]
    out[-1] += total_sum - sum(out)
    return out


def row_max_normalization(tensor):
    return tensor / (tensor.abs().max(dim=-1).values + 1e-9).unsqueeze(-1)
