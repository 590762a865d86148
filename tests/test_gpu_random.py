"""Seeded random sweep over shapes and options against the oracle: ragged lengths, offsets
between query and key positions (including windows that leave rows or whole tiles without
keys), grouped-query K/V, splits, dropout, ALiBi, both dtypes and head dims, and the short
query blocks that go to the decode kernel."""
import numpy as np
import pytest

import gpu_util

pytestmark = pytest.mark.gpu


def _case(seed):
    r = np.random.RandomState(1000 + seed)
    d = int(r.choice([32, 64, 72, 96, 128]))
    Hk = int(r.choice([1, 2, 3]))
    H = Hk * int(r.choice([1, 1, 2, 4]))
    B = int(r.choice([1, 2]))
    short = r.rand() < 0.3
    Nq = int(r.randint(1, 9)) if short else int(r.randint(1, 420))
    Nk = int(r.randint(1, 700))
    causal = bool(r.rand() < 0.5)
    # key position 0 may lie before or after query position 0
    q_pos0 = int(r.choice([0, 0, Nk - Nq if Nk > Nq else 0, int(r.randint(0, 300))]))
    k_pos0 = int(r.choice([0, 0, int(r.randint(0, 200))]))
    window = (-1, -1)
    if r.rand() < 0.4:
        window = (int(r.choice([-1, 0, 17, 128, 300])), int(r.choice([-1, 0, 5, 200])))
    return dict(B=B, H=H, Nq=Nq, Nk=Nk, d=d, dtype=str(r.choice(["bfloat16", "float16"])), seed=seed,
                causal=causal, window=window, alibi=bool(r.rand() < 0.3),
                p_dropout=float(r.choice([0.0, 0.0, 0.1, 0.5])), drop_seed=int(r.randint(0, 1 << 30)),
                offset=int(r.choice([0, 0, 12345])), num_splits=int(r.choice([1, 1, 2, 3, 0])),
                q_pos0=q_pos0, k_pos0=k_pos0, heads_k=Hk)


@pytest.mark.parametrize("seed", range(160))
def test_random_case(seed):
    kw = _case(seed)
    if kw["p_dropout"] > 0 and kw["num_splits"] == 0:
        kw["num_splits"] = 1  # the heuristic's split count decides the dropout streams; pin it
    res = gpu_util.run_case(kw.pop("B"), kw.pop("H"), kw.pop("Nq"), kw.pop("Nk"), kw.pop("d"), **kw)
    gpu_util.assert_close(res, str(_case(seed)))
