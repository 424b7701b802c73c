"""Runs under FLODL_B200_BOUNDS_CHECK=1 (the debug library): a tiny-shape sweep of the kernels that take
indices from device memory must record nothing, and deliberately bad indices must be recorded - as a
{site, index, limit} record on the host, with the access skipped and the context intact."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flodl_b200 import _ext  # noqa: E402

C = _ext.require()
assert C.bounds_check_build(), "this worker needs the bounds-checked library"
dev = "cuda"
C.bounds_report(True)
# ---- clean sweep: ragged and tiny shapes
for rows, cols, V in ((1, 8, 5), (3, 16, 7), (257, 24, 130), (1000, 136, 1000)):
    tgt = torch.randint(0, V, (rows,), device=dev)
    tgt[::3] = -100
    idx, tc, counts = C.compact_targets(tgt, -100)
    x = torch.randn(rows, cols, device=dev).bfloat16()
    xc = torch.empty_like(x)
    C.gather_rows(x, idx, counts, xc)
    dx = torch.zeros_like(x)
    C.scatter_rows(xc, idx, counts, dx)
    logits = torch.randn(rows, V + (8 - V % 8) % 8, device=dev).bfloat16()[:, :V]
    C.softmax_ce(logits, tc, -100, True, False, counts)
    C.softmax_ce(logits, tgt, -100, True, False)
    ids = torch.randint(0, V, (rows,), device=dev)
    dw = torch.zeros(V, cols, device=dev)
    C.embedding_bwd(x, ids, dw, -1)
assert C.bounds_report(True) == [0, 0, 0], "clean inputs must leave the record empty"
# ---- an out-of-range token id: recorded, not dereferenced
ids = torch.tensor([1, 99, 2], device=dev)
dw = torch.zeros(10, 8, device=dev)
C.embedding_bwd(torch.ones(3, 8, device=dev), ids, dw, -1)
site, index, limit = C.bounds_report(True)
assert (site, index, limit) == (101, 99, 10), (site, index, limit)
assert dw.sum().item() == 16.0           # the two valid rows were still accumulated
# ---- a corrupted compaction table
x = torch.randn(16, 8, device=dev).bfloat16()
idx = torch.arange(16, device=dev, dtype=torch.int32)
idx[2] = 500
counts = torch.tensor([4, 16], device=dev, dtype=torch.int32)
xc = torch.zeros_like(x)
C.gather_rows(x, idx, counts, xc)
site, index, limit = C.bounds_report(True)
assert site == 104 and index == 500 and limit == 16, (site, index, limit)
# ---- a label outside the vocabulary
logits = torch.randn(4, 16, device=dev)
C.softmax_ce(logits, torch.tensor([1, 40, 2, 3], device=dev), -100, True, False)
site, index, limit = C.bounds_report(True)
assert (site, index, limit) == (201, 40, 16), (site, index, limit)
assert torch.ones(4, device=dev).sum().item() == 4.0      # the context is still usable
print("BOUNDS_OK")
