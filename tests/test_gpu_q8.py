"""8-bit affine Linear and embedding lookup (the reference's LM head and token embedding format) against the fixture made
by the reference's own linear_big / linear_rows and against the numpy restatement, through the C ABI."""
import numpy as np
import pytest

from ijah_b200 import packgen
from oracle import opref_port as O
from oracle import c_oracle as CO
from tests.helpers import PFX, q8_parts, q8_small, rel_max, small_pack

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    import torch
    assert torch.cuda.is_available()
    from ijah_b200 import engine as E
    return E.Engine()


def test_q8_head_and_embedding_match_reference_fixture(eng):
    import torch
    from ijah_b200 import engine as E
    t, g = q8_small()
    head = E.Q8Linear(eng, *q8_parts(t, "language_model.lm_head"))
    y = head(torch.from_numpy(g["x"]).cuda()).cpu().numpy()
    assert rel_max(y, g["head_y"]) < 1e-5  # activations enter as fp16 hi + lo: f32 accuracy
    assert np.array_equal(y.argmax(1), g["head_y"].argmax(1))
    emb = E.Q8Linear(eng, *q8_parts(t, "language_model.model.embed_tokens"))
    rows = emb.embed(torch.from_numpy(g["ids"]).cuda()).cpu().numpy()
    assert np.array_equal(rows, g["embed_rows"])


@pytest.mark.parametrize("n_out,n_in,group,rows", [(1000, 2560, 64, 1), (4100, 2560, 128, 8), (520, 2048, 64, 19), (136, 320, 64, 50), (264, 5120, 256, 3), (300, 1024, 32, 7), (129, 10240, 64, 12)])
def test_q8_linear_shapes(eng, n_out, n_in, group, rows):
    # ragged output counts (not a multiple of 16 / 128), the reference's input widths and group sizes, more than 16 rows,
    # more inputs than one staged chunk
    import torch
    from ijah_b200 import engine as E
    rng = np.random.default_rng(n_out + rows)
    w, sc, bi = packgen.q8_linear(rng, n_out, n_in, group)
    x = (rng.standard_normal((rows, n_in)) * np.exp(rng.standard_normal((rows, 1)))).astype(np.float32)
    lin = E.Q8Linear(eng, w, sc, bi)
    y = lin(torch.from_numpy(x).cuda()).cpu().numpy()
    want = x.astype(np.float64) @ O.affine_dequant(w, sc, bi).astype(np.float64).T
    assert rel_max(y, want) < 1e-5
    assert np.array_equal(y, lin(torch.from_numpy(x).cuda()).cpu().numpy()), "two runs must be bit-identical"


def test_q8_linear_by_name_and_refusals(eng):
    from ijah_b200 import engine as E
    rng = np.random.default_rng(3)
    w, sc, bi = packgen.q8_linear(rng, 256, 512, 64)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    bufs = [eng.from_numpy(a) for a in (w, sc, bi, x)]
    yb = eng.alloc(3 * 256 * 4)
    ms = eng.run_kernel("q8_linear", bufs + [yb, np.array([512, 256, 64, 3], np.uint32)], reps=2)
    assert ms > 0
    y = yb.numpy(np.float32).reshape(3, 256)
    assert rel_max(y, x @ O.affine_dequant(w, sc, bi).T) < 1e-5
    with pytest.raises(E.EngineError, match="group"):
        eng.run_kernel("q8_linear", bufs + [yb, np.array([512, 256, 48, 3], np.uint32)])


def test_layer_with_q8_shared_expert(eng, tmp_path):
    # a layer whose routed experts are EXL3 and whose shared expert is 8-bit affine (a pack whose trunk was not converted):
    # the shared expert against the fixture of the reference's own shared_expert(), the block against routed + gate * shared
    t, g = small_pack()
    qt, qg = q8_small()
    k = int(g["topk"])
    pack = {n: v for n, v in t.items() if ".mlp.shared_expert" not in n}
    for n, v in qt.items():
        if ".layers.3.mlp." in n:
            pack[n.replace(".layers.3.", ".layers.0.")] = v
    packgen.write_pack(tmp_path / "pack", pack, {"num_experts_per_tok": k}, shards=3, misalign=2)
    p = eng.pack_open(tmp_path / "pack")
    x = qg["x"]
    rows = x.shape[0]
    L = eng.fn_layer(p, 0, rows=rows)
    L.write("mlp_in", x)
    L.run_stage(5)
    y = L.read("mlp_out").reshape(rows, -1)
    sgu = L.read("shared_gu").reshape(rows, 2, -1)
    assert rel_max(sgu[:, 0], qg["sh8_shared_gate_proj"]) < 1e-5 and rel_max(sgu[:, 1], qg["sh8_shared_up_proj"]) < 1e-5
    assert rel_max(L.read("shared_down").reshape(rows, -1), qg["sh8_shared_out"]) < 1e-5
    routed = CO.moe_block_emul({n: v for n, v in t.items() if ".mlp.shared_expert" not in n}, x, top_k=k)
    want = routed["routed"] + qg["sh8_shared_scale"] * qg["sh8_shared_out"]
    assert rel_max(y, want) < 2e-4
    y1 = y.copy()
    for s in (7, 8, 9):
        L.run_dispatch(s)
    assert np.array_equal(L.read("mlp_out").reshape(rows, -1), y1)
    L.free()
    p.close()
