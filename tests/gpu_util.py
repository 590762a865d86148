"""Helpers shared by the GPU parity tests: run the CUDA path through the C ABI on
synthetic inputs and compare with the CPU oracle at the stated tolerances."""
import numpy as np
import torch

import oracle_lib
import synth

# tolerances of the parity bar for 16-bit outputs against the fp32 oracle
O_MAX_ABS = 2e-2
O_MEAN_ABS = 2e-3
LSE_ABS = 1e-3

TORCH_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def to_dev(x, dtype_name):
    return torch.from_numpy(x).to(TORCH_DT[dtype_name]).cuda()


def run_case(B, H, Nq, Nk, d, dtype="bfloat16", seed=0, sigma=1.0, scale=None, causal=False, window=(-1, -1),
             alibi=False, p_dropout=0.0, drop_seed=42, offset=0, num_splits=1, q_pos0=0, k_pos0=0,
             out_dtype=None, rows=None):
    """Returns dict with errors of the CUDA result against the oracle."""
    import flash_attn_b200 as fa
    q, k, v = synth.qkv(seed, B, H, Nq, Nk, d, dtype, sigma)
    slopes = synth.alibi_slopes(H) if alibi else None
    scale = float(scale if scale is not None else 1.0 / np.sqrt(d))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o, lse = fa.flash_attn_forward(
        to_dev(q, dtype), to_dev(k, dtype), to_dev(v, dtype), softmax_scale=scale, causal=causal, window=window,
        alibi_slopes=None if slopes is None else torch.from_numpy(slopes), p_dropout=p_dropout, seed=drop_seed,
        offset=offset, num_splits=num_splits, q_pos0=q_pos0, k_pos0=k_pos0, out_dtype=out_dtype, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device wait timed out: status {int(status.item())}"
    # the split count the library really used decides the dropout stream geometry
    used_splits = num_splits
    if p_dropout > 0 and num_splits != 1:
        used_splits = min(max(1, num_splits), (Nk + 127) // 128)
    want_o, want_lse = oracle_lib.forward(q, k, v, scale, causal=causal, window=window, alibi_slopes=slopes,
                                          p_dropout=p_dropout, seed=drop_seed, offset=offset,
                                          dropout_splits=used_splits, q_pos0=q_pos0, k_pos0=k_pos0, rows=rows)
    got_o = o.float().cpu().numpy()
    got_lse = lse.cpu().numpy()
    if rows is not None:
        got_o = got_o.reshape(-1, d)[rows]
        got_lse = got_lse.reshape(-1)[rows]
    finite = np.isfinite(want_lse)
    res = dict(
        o_max=float(np.abs(got_o - want_o).max()),
        o_mean=float(np.abs(got_o - want_o).mean()),
        lse_max=float(np.abs(got_lse[finite] - want_lse[finite]).max()) if finite.any() else 0.0,
        lse_inf_match=bool(np.array_equal(np.isneginf(got_lse), np.isneginf(want_lse))),
        nan=bool(np.isnan(got_o).any() or np.isnan(got_lse).any()),
    )
    return res


def assert_close(res, what=""):
    msg = f"{what}: {res}"
    assert not res["nan"], msg
    assert res["o_max"] <= O_MAX_ABS, msg
    assert res["o_mean"] <= O_MEAN_ABS, msg
    assert res["lse_max"] <= LSE_ABS, msg
    assert res["lse_inf_match"], msg
