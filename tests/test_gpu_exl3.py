"""CUDA EXL3 decoder and Linear against the oracle, through the C ABI (ne_exl3_dequant, ne_exl3_linear*)."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import c_oracle as CO
from oracle import exl3_codec as X
from oracle import opref_port as O
from tests.helpers import rel_max, small_pack, trunk_linear

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    return E.Engine()


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.mark.parametrize("K", [4, 5, 6, 7, 8])
def test_dequant_is_bit_exact(eng, K):
    from ijah_b200 import engine as E
    rng = np.random.default_rng(10 + K)
    tr, su, sv = packgen.exl3_linear(rng, 512, 272, K)  # 32 x 17 tiles
    lin = E.Exl3Linear(eng, tr, su, sv)
    got = lin.dequant().cpu().numpy()
    want = X.decode_inner(tr).astype(np.float16)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_dequant_all_codewords(eng):
    # a K=8 tile stream whose windows sweep the codebook: every 15-bit state appears
    from ijah_b200 import engine as E
    rng = np.random.default_rng(3)
    tr = rng.integers(0, 1 << 16, (64, 64, 128), dtype=np.uint16)
    seen = np.unique(X.tile_codewords(tr) & 0x7FFF).size
    assert seen > 32000
    lin = E.Exl3Linear(eng, tr, np.ones(1024, np.float16), np.ones(1024, np.float16))
    assert np.array_equal(lin.dequant().cpu().numpy().view(np.uint16), CO.decode_inner(tr).astype(np.float16).view(np.uint16))


CASES = [  # (in, out, K, rows)
    (2048, 768, 5, 1),     # the single-layer configuration
    (2048, 768, 5, 16), (768, 2048, 5, 4), (2048, 768, 4, 2), (2048, 4096, 6, 1), (2048, 4096, 6, 8),
    (2048, 512, 8, 32), (4096, 2048, 8, 1), (4096, 2048, 6, 32), (2048, 512, 7, 3),
    (320, 48, 6, 5),       # Hadamard 64 in / 16 out, one partial column group
    (256, 1040, 5, 1),     # out Hadamard 16, ragged last column group
    (96, 160, 8, 64),      # Hadamard 32 / 32, 64 rows
]


@pytest.mark.parametrize("n_in,n_out,K,rows", CASES)
def test_linear_matches_oracle(eng, n_in, n_out, K, rows):
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(n_in + n_out + K + rows)
    tr, su, sv = packgen.exl3_linear(rng, n_in, n_out, K)
    x = rng.standard_normal((rows, n_in))
    x[:, rng.integers(0, n_in, 4)] *= 20.0  # a few outlier channels, as the reference's kernel check does
    x = x.astype(np.float16).astype(np.float32)
    lin = E.Exl3Linear(eng, tr, su, sv)
    y = lin(torch.from_numpy(x).cuda()).cpu().numpy()
    y_emul = CO.linear_emul(tr, su, sv, x)
    # tolerance of the reference's kernel check (tests/trunk6/check_kernels.py: 5e-5 vs the kernel arithmetic)
    assert rel_l2(y, y_emul) < 5e-5, rel_l2(y, y_emul)
    if n_in * n_out <= 2048 * 768:
        # acceptance bound for layer outputs: max-abs within 2e-3 of the fp32/f64 reference
        assert rel_max(y, O.exl3_linear_exact(x, tr, su, sv)) < 2e-3
    y2 = lin(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(y, y2), "two runs must be bit-identical"
    yh = lin.forward_host(x)
    assert np.array_equal(y, yh)


def test_trunk_fixture_from_reference(eng):
    import torch
    from ijah_b200 import engine as E
    t, g = small_pack()
    x = g["x"]
    for layer in (0, 1):
        for proj in ("q", "k", "v", "o"):
            o = trunk_linear(t, layer, proj)
            xin = x if o.inner.shape[0] == x.shape[1] else np.tile(x, (1, o.inner.shape[0] // x.shape[1]))
            lin = E.Exl3Linear(eng, o.trellis, o.suh, o.svh)
            y = lin(torch.from_numpy(np.ascontiguousarray(xin)).cuda()).cpu().numpy()
            assert rel_max(y, g[f"trunk_L{layer}_{proj}_y"]) < 2e-3


def test_linearity_at_full_size(eng):
    # size-independent property at the trunk's largest shape: f(a x1 + x2) = a f(x1) + f(x2) up to fp16 preparation
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(0)
    tr, su, sv = packgen.exl3_linear(rng, 4096, 2048, 6)
    lin = E.Exl3Linear(eng, tr, su, sv)
    x1 = torch.from_numpy(rng.standard_normal((1, 4096)).astype(np.float32)).cuda()
    x2 = torch.from_numpy(rng.standard_normal((1, 4096)).astype(np.float32)).cuda()
    lhs = lin(2.0 * x1 + x2)
    rhs = 2.0 * lin(x1) + lin(x2)
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) < 2e-3


def test_bad_arguments_are_refused(eng):
    import ctypes as C
    from ijah_b200 import engine as E
    rng = np.random.default_rng(0)
    tr, su, sv = packgen.exl3_linear(rng, 256, 128, 5)
    lin = E.Exl3Linear(eng, tr, su, sv)
    import torch
    x = torch.zeros((65, 256), device="cuda")
    with pytest.raises(E.EngineError, match="rows"):
        lin(x)
    bad = E.Exl3WeightC(lin.c.trellis, lin.c.suh, lin.c.svh, 250, 128, 5)
    y = torch.zeros((1, 128), device="cuda")
    assert eng.lib.ne_exl3_linear(C.byref(bad), C.c_void_p(x.data_ptr()), 1, C.c_void_p(y.data_ptr()), None) == -1
    assert "multiples of 16" in eng.last_error()
    assert eng.lib.ne_device_wait_status() == 0


@pytest.mark.parametrize("rows", [1, 8, 32])
def test_linears_on_shared_rows_in_one_chain(eng, rows):
    # the q, k, v projections of the trunk configuration (K6, one of them K8) through ne_exl3_linear_multi
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(40 + rows)
    shapes = [(2048, 4096, 6), (2048, 512, 6), (2048, 512, 8), (2048, 320, 5)]
    lins, packs = [], []
    for n_in, n_out, K in shapes:
        tr, su, sv = packgen.exl3_linear(rng, n_in, n_out, K)
        packs.append((tr, su, sv))
        lins.append(E.Exl3Linear(eng, tr, su, sv))
    x = rng.standard_normal((rows, 2048)).astype(np.float16).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    outs = [torch.empty((rows, s[1]), device="cuda") for s in shapes]
    E.linear_multi(eng, lins, xd, outs)
    for lin, pk, o in zip(lins, packs, outs):
        got = o.cpu().numpy()
        want = CO.linear_emul(*pk, x)
        assert np.linalg.norm(got - want) / np.linalg.norm(want) < 5e-5
        assert rel_max(got, lin(xd).cpu().numpy()) < 1e-5
    again = [torch.empty_like(o) for o in outs]
    E.linear_multi(eng, lins, xd, again)
    assert all(torch.equal(a, b) for a, b in zip(outs, again)), "two runs must be bit-identical"
    assert eng.lib.ne_device_wait_status() == 0
    with pytest.raises(E.EngineError):  # different input widths
        tr, su, sv = packgen.exl3_linear(rng, 256, 256, 4)
        E.linear_multi(eng, [lins[0], E.Exl3Linear(eng, tr, su, sv)], xd, outs[:2])
