"""The opt-in summand product (ne_exl3_set_summand_product(1)): every weight enters the tensor core as its two fp16 summands and
their sum is not rounded to fp16 first. Checked against the emulation of exactly that arithmetic at the same tolerances
as the default (exact) product against its own, and against the float64 reference at the acceptance bound."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import c_oracle as CO
from oracle import opref_port as O
from tests.helpers import MoeView, rel_max

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.fixture()
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    e = E.Engine()
    assert e.lib.ne_exl3_set_summand_product(1) == 0, "the exact product is the default"
    assert e.lib.ne_exl3_set_summand_product(-1) == 1
    yield e
    assert e.lib.ne_exl3_set_summand_product(0) == 1


@pytest.mark.parametrize("n_in,n_out,K,rows", [(2048, 768, 5, 4), (768, 2048, 5, 16), (512, 1024, 6, 1), (1024, 512, 8, 40)])
def test_linear_in_both_modes(eng, n_in, n_out, K, rows):
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(n_in + K + rows)
    tr, su, sv = packgen.exl3_linear(rng, n_in, n_out, K)
    x = rng.standard_normal((rows, n_in)).astype(np.float16).astype(np.float32)
    lin = E.Exl3Linear(eng, tr, su, sv)
    xd = torch.from_numpy(x).cuda()
    y_sum = lin(xd).cpu().numpy()
    eng.lib.ne_exl3_set_summand_product(0)
    y_exact = lin(xd).cpu().numpy()
    eng.lib.ne_exl3_set_summand_product(1)
    assert rel_l2(y_sum, CO.linear_emul(tr, su, sv, x, summands=True)) < 5e-5
    assert rel_l2(y_exact, CO.linear_emul(tr, su, sv, x, summands=False)) < 5e-5
    # the two arithmetics differ by the fp16 rounding of each weight: visible, and far inside the acceptance bound
    assert 1e-5 < rel_l2(y_sum, y_exact) < 1e-3
    ref = O.exl3_linear_exact(x, tr, su, sv)
    assert rel_max(y_sum, ref) < 2e-3 and rel_max(y_exact, ref) < 2e-3


def test_moe_block_summand_product(eng):
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(77)
    t = packgen.moe_layer(rng, hidden=512, inter=256, experts=32)
    x = rng.standard_normal((5, 512)).astype(np.float16).astype(np.float32)
    blk = E.MoeBlock(eng, t, top_k=4, max_rows=8)
    y = blk.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    want = CO.moe_block_emul(t, x, top_k=4, want_gu=True, summands=True)
    ids, _ = blk.route(5)
    assert np.array_equal(ids, want["ids"])
    assert rel_max(blk.experts_gu(5), want["experts_gu"]) < 2e-4
    assert rel_max(y, want["out"]) < 2e-4
    mv = MoeView(t)
    assert rel_max(y, O.moe_block_exact(x, mv.router, mv.sgate, mv.expert, mv.shared, 4)["out"]) < 2e-3
