"""The C restatement (oracle/exl3_oracle.c) against the numpy one. CPU only."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import c_oracle as CO
from oracle import exl3_codec as X
from oracle import opref_port as O
from tests.helpers import MoeView, rel_max, small_pack


@pytest.mark.parametrize("K", [4, 5, 6, 7, 8])
def test_c_decode_and_linear_match_numpy(K):
    rng = np.random.default_rng(K)
    tr, su, sv = packgen.exl3_linear(rng, 320, 48, K)  # Hadamard 64 in, 16 out
    assert np.array_equal(CO.decode_inner(tr), X.decode_inner(tr))
    x = rng.standard_normal((3, 320)).astype(np.float32)
    assert rel_max(CO.linear_emul(tr, su, sv, x), O.exl3_linear_emul(x, tr, su, sv)) < 1e-6


def test_c_moe_block_matches_numpy_and_reference_fixture():
    t, g = small_pack()
    mv = MoeView(t)
    k = int(g["topk"])
    r = CO.moe_block_emul(t, g["x"], top_k=k, want_gu=True)
    n = O.moe_block_emul(g["x"], mv.router, mv.sgate, mv.expert, mv.shared, k)
    assert np.array_equal(r["ids"], g["ids"])
    assert rel_max(r["out"], n["out"]) < 1e-5
    assert rel_max(r["experts_gu"], n["experts_gu"]) < 1e-5
    assert rel_max(r["out"], g["block_out"]) < 2e-3
