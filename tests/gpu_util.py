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
             out_dtype=None, rows=None, heads_k=None, host=False, launch_index=0):
    """Returns dict with errors of the CUDA result against the oracle.  heads_k < H runs
    grouped-query attention (the oracle sees K/V repeated per query head); host=True goes
    through the host-buffer entry point."""
    import flash_attn_b200 as fa
    q, k, v = synth.qkv(seed, B, H, Nq, Nk, d, dtype, sigma)
    k_dev, v_dev = k, v
    if heads_k is not None and heads_k != H:
        k_dev = np.ascontiguousarray(k[:, :heads_k])
        v_dev = np.ascontiguousarray(v[:, :heads_k])
        k = np.repeat(k_dev, H // heads_k, axis=1)
        v = np.repeat(v_dev, H // heads_k, axis=1)
    slopes = synth.alibi_slopes(H) if alibi else None
    scale = float(scale if scale is not None else 1.0 / np.sqrt(d))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if host:
        pin = lambda x: torch.from_numpy(x).to(TORCH_DT[dtype]).pin_memory()
        o, lse = fa.flash_attn_forward_host(
            pin(q), pin(k_dev), pin(v_dev), softmax_scale=scale, causal=causal, window=window,
            alibi_slopes=None if slopes is None else torch.from_numpy(slopes), p_dropout=p_dropout, seed=drop_seed,
            offset=offset, num_splits=num_splits, out_dtype=out_dtype)
    else:
        o, lse = fa.flash_attn_forward(
            to_dev(q, dtype), to_dev(k_dev, dtype), to_dev(v_dev, dtype), softmax_scale=scale, causal=causal,
            window=window, alibi_slopes=None if slopes is None else torch.from_numpy(slopes), p_dropout=p_dropout,
            seed=drop_seed, offset=offset, num_splits=num_splits, q_pos0=q_pos0, k_pos0=k_pos0, out_dtype=out_dtype,
            status=status, launch_index=launch_index)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device wait timed out: status {int(status.item())}"
    # the split count the library really used decides the dropout stream geometry
    used_splits = num_splits
    if p_dropout > 0 and num_splits != 1:
        used_splits = min(max(1, num_splits), (Nk + 127) // 128)
    want_o, want_lse = oracle_lib.forward(q, k, v, scale, causal=causal, window=window, alibi_slopes=slopes,
                                          p_dropout=p_dropout, seed=drop_seed, offset=offset,
                                          dropout_splits=used_splits, q_pos0=q_pos0, k_pos0=k_pos0, rows=rows,
                                          launch_index=launch_index)
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


def check_sampled_units(q, k, v, o, lse, units, rows_of_unit, scale, causal=False, window=(-1, -1), slopes=None,
                        q_pos0=0, k_pos0=0):
    """Oracle comparison for tensors that live on the GPU (shapes too large to generate or check whole on the
    host): for every sampled (batch, head) unit its K/V and the sampled query rows are copied to the host and
    the oracle evaluates those rows.  q/o [B,H,Nq,d], k/v [B,H,Nk,d] CUDA tensors; `units` flat b*H+h indices;
    `rows_of_unit(u)` -> row indices inside the unit.  Returns the same error dict as run_case."""
    B, H, Nq, d = q.shape
    o_err, lse_err, n, o_sum = 0.0, 0.0, 0, 0.0
    inf_ok, nan = True, False
    for u in units:
        b, h = divmod(int(u), H)
        rows = np.asarray(sorted(set(int(r) for r in rows_of_unit(u))), dtype=np.int64)
        qh = q[b, h].float().cpu().numpy()[None, None]
        kh = k[b, h % k.shape[1] if k.shape[1] == H else h // (H // k.shape[1])].float().cpu().numpy()[None, None]
        vh = v[b, h % v.shape[1] if v.shape[1] == H else h // (H // v.shape[1])].float().cpu().numpy()[None, None]
        want_o, want_lse = oracle_lib.forward(qh, kh, vh, scale, causal=causal, window=window,
                                              alibi_slopes=None if slopes is None else slopes[h:h + 1],
                                              q_pos0=q_pos0, k_pos0=k_pos0, rows=rows)
        got_o = o[b, h].float().cpu().numpy()[rows]
        got_lse = lse[b, h].cpu().numpy()[rows]
        fin = np.isfinite(want_lse)
        o_err = max(o_err, float(np.abs(got_o - want_o).max()))
        o_sum += float(np.abs(got_o - want_o).sum())
        n += got_o.size
        if fin.any():
            lse_err = max(lse_err, float(np.abs(got_lse[fin] - want_lse[fin]).max()))
        inf_ok = inf_ok and bool(np.array_equal(np.isneginf(got_lse), np.isneginf(want_lse)))
        nan = nan or bool(np.isnan(got_o).any() or np.isnan(got_lse).any())
    return dict(o_max=o_err, o_mean=o_sum / max(n, 1), lse_max=lse_err, lse_inf_match=inf_ok, nan=nan)
