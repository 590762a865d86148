"""Key blocks that arrive one launch at a time: every launch merges its result into the caller's running
(O, LSE) pair in the kernel epilogue (fa_fwd_params.accum_o).  The merged result over uneven blocks must match the
oracle on the whole key sequence; dropout masks of later launches of a loop (launch_index) must match the oracle's
on the tiled and the decode kernel."""
import numpy as np
import pytest
import torch

import gpu_util
import oracle_lib
import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", [
    dict(B=1, H=2, Nq=600, blocks=(256, 384, 137), d=128, dtype="bfloat16", causal=True),    # two-tile CTAs
    dict(B=2, H=3, Nq=100, blocks=(200, 300, 37), d=64, dtype="float16", causal=False),      # one-tile CTAs
    dict(B=1, H=4, Nq=300, blocks=(128, 128, 128, 128), d=128, dtype="bfloat16", causal=True, window=(150, 0), alibi=True),
    dict(B=1, H=2, Nq=260, blocks=(500,), d=96, dtype="float16", causal=False),               # first and last in one launch
    dict(B=1, H=2, Nq=5, blocks=(300, 200), d=128, dtype="bfloat16", causal=True),            # short query: tiled kernel in this mode
])
def test_blocks_merged_in_the_epilogue_match_the_oracle(case):
    import flash_attn_b200 as fa
    B, H, Nq, d = case["B"], case["H"], case["Nq"], case["d"]
    Nk = sum(case["blocks"])
    q_pos0 = Nk - Nq if case["causal"] else 0  # bottom-right aligned: every row sees some key of the first block
    qn, kn, vn = synth.qkv(60, B, H, Nq, Nk, d, case["dtype"], 0.7)
    q, k, v = (gpu_util.to_dev(x, case["dtype"]) for x in (qn, kn, vn))
    slopes = synth.alibi_slopes(H) if case.get("alibi") else None
    window = case.get("window", (-1, -1))
    acc = (torch.full((B, H, Nq, d), float("nan"), device="cuda"), torch.full((B, H, Nq), float("nan"), device="cuda"))
    pos, out = 0, None
    for i, n in enumerate(case["blocks"]):
        out = fa.flash_attn_forward(q, k[:, :, pos:pos + n].contiguous(), v[:, :, pos:pos + n].contiguous(),
                                    causal=case["causal"], window=window,
                                    alibi_slopes=None if slopes is None else torch.from_numpy(slopes), q_pos0=q_pos0, k_pos0=pos,
                                    accum=acc, accum_first=i == 0, accum_final=i + 1 == len(case["blocks"]))
        assert (out[0] is None) == (i + 1 < len(case["blocks"]))
        pos += n
    torch.cuda.synchronize()
    o, lse = out
    want_o, want_lse = oracle_lib.forward(qn, kn, vn, d ** -0.5, causal=case["causal"], window=window, alibi_slopes=slopes,
                                          q_pos0=q_pos0)
    fin = np.isfinite(want_lse)
    res = dict(o_max=float(np.abs(o.float().cpu().numpy() - want_o).max()),
               o_mean=float(np.abs(o.float().cpu().numpy() - want_o).mean()),
               lse_max=float(np.abs(lse.cpu().numpy()[fin] - want_lse[fin]).max()),
               lse_inf_match=bool(np.array_equal(np.isneginf(lse.cpu().numpy()), np.isneginf(want_lse))),
               nan=bool(torch.isnan(o.float()).any().item()))
    gpu_util.assert_close(res, str(case))
    # the running LSE equals the final one
    assert torch.equal(acc[1], lse)


def test_rows_that_see_nothing_in_a_block_keep_their_running_result():
    # causal with the second block wholly after the first 128 queries: those rows must come through unchanged
    import flash_attn_b200 as fa
    B, H, Nq, d = 1, 2, 256, 128
    qn, kn, vn = synth.qkv(61, B, H, Nq, 512, d, "bfloat16")
    q, k, v = (gpu_util.to_dev(x, "bfloat16") for x in (qn, kn, vn))
    acc = (torch.empty((B, H, Nq, d), device="cuda"), torch.empty((B, H, Nq), device="cuda"))
    fa.flash_attn_forward(q, k[:, :, :256].contiguous(), v[:, :, :256].contiguous(), causal=True, accum=acc, accum_first=True)
    o, lse = fa.flash_attn_forward(q, k[:, :, 256:].contiguous(), v[:, :, 256:].contiguous(), causal=True, k_pos0=256,
                                   accum=acc, accum_final=True)  # no row sees any of these keys
    want_o, want_lse = oracle_lib.forward(qn, kn[:, :, :256], vn[:, :, :256], d ** -0.5, causal=True)
    assert np.abs(o.float().cpu().numpy() - want_o).max() <= gpu_util.O_MAX_ABS
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= gpu_util.LSE_ABS


def test_accumulate_mode_rejects_splits():
    import flash_attn_b200 as fa
    from flash_attn_b200 import _lib
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 1, 1024, 64, dtype=torch.float16, device="cuda")
    acc = (torch.empty((1, 1, 128, 64), device="cuda"), torch.empty((1, 1, 128), device="cuda"))
    with pytest.raises(_lib.FaError) as e:
        fa.flash_attn_forward(q, k, k, num_splits=4, accum=acc, accum_first=True, accum_final=True)
    assert e.value.code == -2


@pytest.mark.parametrize("case", [dict(Nq=384, Nk=384, causal=True, window=(-1, -1), k=2),
                                  dict(Nq=300, Nk=640, causal=False, window=(200, 64), k=1),
                                  dict(Nq=1, Nk=1000, causal=False, window=(-1, -1), k=3, splits=3),   # decode kernel
                                  dict(Nq=256, Nk=512, causal=True, window=(-1, -1), k=1, splits=2, q_pos0=256)])
def test_later_launch_masks_against_the_oracle(case):
    res = gpu_util.run_case(1, 2, case["Nq"], case["Nk"], 128, "bfloat16", seed=62, causal=case["causal"], window=case["window"],
                            p_dropout=0.2, drop_seed=11, num_splits=case.get("splits", 1), q_pos0=case.get("q_pos0", 0),
                            launch_index=case["k"])
    gpu_util.assert_close(res, str(case))
