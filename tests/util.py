"""Helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np
import torch

import oracle

# Probability tolerances of the parity contract.
#   fp32 logits: |a - b| <= 1e-6 + 1e-5 * |b|
#   fp16 logits: 2e-3 relative (plus half a subnormal step of the fp16 output format)
#   bf16 logits: 8e-3 relative (three mantissa bits fewer than fp16)
TOL = {torch.float32: (1e-6, 1e-5), torch.float16: (6e-8, 2e-3), torch.bfloat16: (1e-30, 8e-3)}
ORACLE_DTYPE = {torch.float32: oracle.F32, torch.float16: oracle.F16, torch.bfloat16: oracle.BF16}
to_oracle_array = oracle.to_oracle_array


def oracle_softmax_topk(x: torch.Tensor, k: int, inv_temperature: float = 1.0, value_kind=oracle.VALUE_PROBABILITY):
    return oracle.softmax_topk(to_oracle_array(x), k, inv_temperature, dtype=ORACLE_DTYPE[x.dtype],
                               value_kind=value_kind, sum_mode=oracle.SUM_F64)


def assert_probs_close(got: torch.Tensor, want: np.ndarray, dtype: torch.dtype, what: str = ""):
    atol, rtol = TOL[dtype]
    g = got.detach().float().cpu().numpy().astype(np.float64)
    w = want.astype(np.float64)
    both_nan = np.isnan(g) & np.isnan(w)
    err = np.abs(g - w)
    ok = (err <= atol + rtol * np.abs(w)) | both_nan
    if not ok.all():
        bad = np.argwhere(~ok)[0]
        raise AssertionError(f"{what}: probability mismatch at {tuple(bad)}: got {g[tuple(bad)]!r} want {w[tuple(bad)]!r} "
                             f"(atol {atol}, rtol {rtol}); {np.count_nonzero(~ok)} bad of {ok.size}")


def assert_indices_equal(got: torch.Tensor, want: np.ndarray, what: str = ""):
    g = got.detach().cpu().numpy().astype(np.int64)
    if not np.array_equal(g, want.astype(np.int64)):
        bad = np.argwhere(g != want)[0]
        raise AssertionError(f"{what}: index mismatch at {tuple(bad)}: got {g[tuple(bad)]} want {want[tuple(bad)]}; "
                             f"{np.count_nonzero(g != want)} bad of {g.size}")


def check_fused(x_cpu: torch.Tensor, k: int, inv_temperature: float = 1.0, what: str = "", **kw):
    """Runs the CUDA fused op on x (moved to the GPU) and compares with the oracle."""
    from vkop_b200 import capi

    xg = x_cpu.cuda()
    vals, idx = capi.softmax_topk(xg, k, inv_temperature, **kw)
    torch.cuda.synchronize()
    wv, wi = oracle_softmax_topk(x_cpu, k, inv_temperature)
    assert_indices_equal(idx, wi, what)
    assert_probs_close(vals, wv, x_cpu.dtype, what)
    return vals, idx


def merge_packets_reference(packets, k: int, full_logits: np.ndarray, dtype: int):
    """Numpy statement of the packet merge (test-side): packets = list of (m, s, keys, idx, count) per shard, as
    oracle.shard_packet returns them.  Returns (values f32 [rows,k], indices i64 [rows,k])."""
    rows = packets[0][0].shape[0]
    vals = np.empty((rows, k), np.float32)
    idxs = np.empty((rows, k), np.int64)
    for r in range(rows):
        M, S = oracle.merge_stats(np.array([p[0][r] for p in packets]), np.array([p[1][r] for p in packets]))
        cand = []
        for m, s, keys, idx, cnt in packets:
            cand += [(-int(keys[r, j]), int(idx[r, j])) for j in range(int(cnt[r]))]
        cand.sort()
        best = cand[:k]
        idxs[r] = [c[1] for c in best]
        row = full_logits[r:r + 1, idxs[r]]
        if dtype == oracle.F32:
            x = row.astype(np.float32)
        elif dtype == oracle.F16:
            x = row.view(np.float16).astype(np.float32)
        else:
            x = (row.astype(np.uint32) << 16).view(np.float32)
        vals[r] = (np.exp(x.astype(np.float64)[0] - np.float64(M)) / S).astype(np.float32)
    return vals, idxs
