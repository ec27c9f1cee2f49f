"""The CPU oracle against vectors produced by the reference itself (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import hsa_oracle as orc
from tests.conftest import rel_err

WEIGHT_NAMES = ["Wq_y.weight", "Wk_y.weight", "Wv_y.weight", "out_proj_y.weight", "out_proj_y.bias",
                "Wq_x.weight", "Wk_x.weight", "Wv_x.weight", "out_proj_x.weight", "out_proj_x.bias"]

# first 32 hex digits of sha256 over the three tables, generated from the reference's builder
DIGESTS = {
    (2, 1): "ba5b14448b0605cab1a8ced176a20978", (2, 0): "f9ec7d928d1a4441f538202b62fde9ca",
    (4, 1): "7e3ea3690f9419f6a0824a8930497500", (4, 0): "5498e64d4a10fbf55b1ed88c0d242a6a",
    (8, 1): "3c82bad0e3b62674de259a25c2c307f2", (8, 0): "85abaef93f4666eed6382dac03f453ab",
    (64, 1): "19da5e81e17aa5f18a72abea0f67c35d", (64, 0): "ee1484dabb1dd9dffd7b96ccde9e0c41",
    (512, 1): "32d1520016199dda9581f9199a8553f3", (512, 0): "f8ec0fda52fb802abc9da991aff41d23",
    (4096, 1): "3c89ab759b2fe43d6e90ffea2e588a4a", (4096, 0): "e9f1a06d57aad24df015437906dba5e4",
}


def test_topology_tables_exact(golden):
    g = golden("topology.npz")
    for N in (2, 4, 8, 16, 32):
        for c in (1, 0):
            t = orc.build_tree_topology(N, bool(c))
            tag = f"N{N}_c{c}"
            assert np.array_equal(t["forward_idx"], g[f"idx_{tag}"])
            assert np.array_equal(t["forward_mask"], g[f"mask_{tag}"])
            assert np.array_equal(t["backward_gather"], g[f"gather_{tag}"])


def test_topology_known_answer_n8():
    t = orc.build_tree_topology(8, True)
    assert t["forward_idx"].tolist() == [[1, 9, 13], [0, 9, 13], [3, 8, 13], [2, 8, 13],
                                         [5, 11, 12], [4, 11, 12], [7, 10, 12], [6, 10, 12]]
    rows = {r: tuple(v) for r, v in enumerate(t["backward_gather"].tolist()) if v[0] != -1}
    assert rows == {0: (1, 2, 0), 2: (3, 4, 0), 4: (5, 6, 0), 6: (7, 8, 0),
                    8: (2, 4, 1), 10: (6, 8, 1), 12: (4, 8, 2)}


def test_topology_digests(golden):
    g = golden("topology.npz")
    stored = {(int(n), int(c)): str(h) for n, c, h in zip(g["digest_N"], g["digest_causal"], g["digest_hex"])}
    for key, hexd in DIGESTS.items():
        assert stored[key] == hexd
    for (N, c), hexd in stored.items():
        if N > 4096:
            continue                       # the explicit climb is O(N log N) python; 32768 is covered on the GPU
        assert orc.topology_digest(orc.build_tree_topology(N, bool(c))) == hexd


def test_span_input_y(golden):
    g = golden("span_input_y.npz")
    for name in "abcd":
        y = orc.generate_span_input_Y(torch.from_numpy(g[f"x_{name}"]))
        assert np.array_equal(y.numpy(), g[f"y_{name}"])
    y = orc.generate_span_input_Y(torch.from_numpy(g["x_bf16"]).to(torch.bfloat16))
    assert np.array_equal(y.float().numpy(), g["y_bf16"])
    assert orc.generate_span_input_Y(torch.zeros(1, 1, 4)) is None


def _load_layer(g, tag):
    B, N, H, Dh, R, seed, sub = (int(v) for v in g[f"{tag}.meta"])
    m = orc.HierarchicalAttentionOracle(H * Dh, H, dropout=0.0, window_size=R).eval()
    m.load_state_dict({k: torch.from_numpy(g[f"{tag}.{k}"]) for k in WEIGHT_NAMES})
    return m, (B, N, H, Dh, R)


@pytest.mark.parametrize("tag", ["tiny", "small", "wide_window"])
def test_layer_against_eager_reference(golden, tag):
    g = golden("layer_eager.npz")
    m, (B, N, H, Dh, R) = _load_layer(g, tag)
    x = torch.from_numpy(g[f"{tag}.x"])
    gy = torch.from_numpy(g[f"{tag}.gy"])
    go = torch.from_numpy(g[f"{tag}.go"])
    xa = x.clone().requires_grad_()
    ya = orc.generate_span_input_Y(x).requires_grad_()
    y1 = m.cross_update_Y(xa, ya)
    y1.backward(gy)
    assert rel_err(y1.detach(), g[f"{tag}.y_new"]) < 1e-5
    assert rel_err(xa.grad, g[f"{tag}.cuy_grad_x"]) < 1e-5
    assert rel_err(ya.grad, g[f"{tag}.cuy_grad_y"]) < 1e-5
    for c in (1, 0):
        xb = x.clone().requires_grad_()
        yb = torch.from_numpy(g[f"{tag}.y_new"]).clone().requires_grad_()
        o = m(xb, xb, xb, y=yb, mask=torch.ones(B, N) if c else None)
        o.backward(go)
        assert rel_err(o.detach(), g[f"{tag}.out_c{c}"]) < 1e-5
        assert rel_err(xb.grad, g[f"{tag}.fwd_grad_x_c{c}"]) < 1e-5
        assert rel_err(yb.grad, g[f"{tag}.fwd_grad_y_c{c}"]) < 1e-5


def config1_inputs(g):
    """Oracle layer, inputs and upstream gradients of the fp32 case B2 H4 N512 Dh64 R16, all read from the fixture."""
    m, _ = _load_layer(g, "config1")
    return m, torch.from_numpy(g["config1.x"]), torch.from_numpy(g["config1.gy"]), torch.from_numpy(g["config1.go"])


def test_b2_h4_n512_fp32_against_eager_reference(golden):
    g = golden("layer_config1.npz")
    m, x, gy, go = config1_inputs(g)
    sub = int(g["config1.meta"][6])
    xa = x.clone().requires_grad_()
    ya = orc.generate_span_input_Y(x).requires_grad_()
    y1 = m.cross_update_Y(xa, ya)
    y1.backward(gy)
    assert rel_err(y1.detach()[:, ::sub], g["config1.y_new"]) < 1e-5
    assert rel_err(xa.grad[:, ::sub], g["config1.cuy_grad_x"]) < 1e-5
    assert rel_err(ya.grad[:, ::sub], g["config1.cuy_grad_y"]) < 1e-5
    xb = x.clone().requires_grad_()
    yb = y1.detach().clone().requires_grad_()
    o = m(xb, xb, xb, y=yb, mask=torch.ones(2, 512))
    o.backward(go)
    assert rel_err(o.detach()[:, ::sub], g["config1.out_c1"]) < 1e-5
    assert rel_err(xb.grad[:, ::sub], g["config1.fwd_grad_x_c1"]) < 1e-5
    assert rel_err(yb.grad[:, ::sub], g["config1.fwd_grad_y_c1"]) < 1e-5


def test_ops_against_triton_interpreter(golden):
    g = golden("triton_ops.npz")
    names = ("Qp", "Kp", "Vp", "Kc", "Vc")
    ts = [torch.from_numpy(g[f"parent.{n}"]).requires_grad_() for n in names]
    o = orc.build_parent_nodes(*ts)
    o.backward(torch.from_numpy(g["parent.go"]))
    assert rel_err(o.detach(), g["parent.out"]) < 1e-5
    for n, t in zip(names, ts):
        assert rel_err(t.grad, g[f"parent.d{n}"]) < 1e-5
    for tag in ("span_a", "span_b", "span_r0"):
        B, N, H, D, R = (int(v) for v in g[f"{tag}.meta"])
        for c in (1, 0):
            q, k, v = (torch.from_numpy(g[f"{tag}.{n}"]).requires_grad_() for n in "QKV")
            o = orc.hierarchical_attention(q, k, v, R, bool(c))
            o.backward(torch.from_numpy(g[f"{tag}.go"]))
            assert rel_err(o.detach(), g[f"{tag}.out_c{c}"]) < 1e-5
            assert rel_err(q.grad, g[f"{tag}.dQ_c{c}"]) < 1e-5
            assert rel_err(k.grad, g[f"{tag}.dK_c{c}"]) < 1e-5
            assert rel_err(v.grad, g[f"{tag}.dV_c{c}"]) < 1e-5


def test_logits_ops_against_reference(golden):
    g = golden("logits_ops.npz")
    for tag in ("w_a", "w_b", "w_r0"):
        B, N, H, D, R = (int(v) for v in g[f"{tag}.meta"])
        for c in (1, 0):
            w = orc.span_logits(torch.from_numpy(g[f"{tag}.Q"]), torch.from_numpy(g[f"{tag}.K"]), R, bool(c), weights=True)
            assert rel_err(w, g[f"{tag}.weights_c{c}"]) < 1e-5
            lg = orc.span_logits(torch.from_numpy(g[f"{tag}.Q"]), torch.from_numpy(g[f"{tag}.K"]), R, bool(c))
            assert bool(((lg == float("-inf")) == (torch.from_numpy(g[f"{tag}.weights_c{c}"]) == 0)).all())
    B, N, H, D = (int(v) for v in g["v1.meta"])
    _, cross = orc.sibling_logits(torch.from_numpy(g["v1.ALL_Q"]), torch.from_numpy(g["v1.ALL_K"]), H, D, N)
    assert rel_err(cross, g["v1.RES_CROSS"]) < 1e-5
