"""Generate the golden vectors under tests/golden/ from the reference project itself.

Run where the reference checkout is mounted (its directory: HSA_REFERENCE_DIR, default `REF` below):

    python tests/golden/make_golden.py

It imports, unmodified,
  * hierarchical_attention.build_tree_topology / generate_span_input_Y (pure torch),
  * the eager layer HierarchicalSparseAttentionRef from
    hierarchical_attention_project/Hierarchical_Attention_Triton_Test.py,
  * the package ops build_parent_nodes / hierarchical_attention, executed on the CPU by
    the Triton interpreter (TRITON_INTERPRET=1),
feeds them seeded inputs and stores inputs and outputs in small .npz files.  The tests
never need the reference again: they read these files.
"""
import os

os.environ["TRITON_INTERPRET"] = "1"

import hashlib
import importlib.util
import sys

import numpy as np
import torch

REF = os.environ.get("HSA_REFERENCE_DIR", "/root/reference")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REF)

from hierarchical_attention import (  # noqa: E402  (the reference package)
    build_parent_nodes, build_tree_topology, generate_span_input_Y, hierarchical_attention)

_spec = importlib.util.spec_from_file_location(
    "ref_eager", os.path.join(REF, "hierarchical_attention_project", "Hierarchical_Attention_Triton_Test.py"))
ref_eager = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(ref_eager)

WEIGHT_NAMES = ["Wq_y.weight", "Wk_y.weight", "Wv_y.weight", "out_proj_y.weight", "out_proj_y.bias",
                "Wq_x.weight", "Wk_x.weight", "Wv_x.weight", "out_proj_x.weight", "out_proj_x.bias"]


def digest(t):
    h = hashlib.sha256()
    h.update(t["forward_idx"].to(torch.int32).contiguous().numpy().tobytes())
    h.update(t["forward_mask"].to(torch.bool).contiguous().numpy().tobytes())
    h.update(t["backward_gather"].to(torch.int32).contiguous().numpy().tobytes())
    return h.hexdigest()[:32]


def topology():
    out = {}
    for N in (2, 4, 8, 16, 32):
        for causal in (True, False):
            t = build_tree_topology(N, is_causal=causal, device="cpu")
            tag = f"N{N}_c{int(causal)}"
            out[f"idx_{tag}"] = t["forward_idx"].numpy().astype(np.int32)
            out[f"mask_{tag}"] = t["forward_mask"].numpy().astype(np.bool_)
            out[f"gather_{tag}"] = t["backward_gather"].numpy().astype(np.int32)
    digs = []
    for N in (2, 4, 8, 16, 64, 512, 2048, 4096, 32768):
        for causal in (True, False):
            digs.append((N, int(causal), digest(build_tree_topology(N, is_causal=causal, device="cpu"))))
    out["digest_N"] = np.array([d[0] for d in digs], dtype=np.int64)
    out["digest_causal"] = np.array([d[1] for d in digs], dtype=np.int64)
    out["digest_hex"] = np.array([d[2] for d in digs])
    np.savez_compressed(os.path.join(HERE, "topology.npz"), **out)


def span_y():
    out = {}
    g = torch.Generator().manual_seed(11)
    for name, shape in (("a", (2, 16, 8)), ("b", (1, 12, 5)), ("c", (3, 64, 24)), ("d", (1, 2, 4))):
        x = torch.randn(*shape, generator=g)
        out[f"x_{name}"] = x.numpy()
        out[f"y_{name}"] = generate_span_input_Y(x).numpy()
    xb = torch.randn(2, 32, 16, generator=g).to(torch.bfloat16)
    out["x_bf16"] = xb.float().numpy()
    out["y_bf16"] = generate_span_input_Y(xb).float().numpy()
    np.savez_compressed(os.path.join(HERE, "span_input_y.npz"), **out)


def layer_case(tag, B, N, H, Dh, R, seed, out, subsample=1):
    """Eager twin: cross_update_Y and forward (+ gradients), causal and non-causal."""
    dim = H * Dh
    torch.manual_seed(seed)
    ref = ref_eager.HierarchicalSparseAttentionRef(dim, H, dropout=0.0, window_size=R).eval()
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(B, N, dim, generator=g)
    y0 = generate_span_input_Y(x)
    gy = torch.randn(B, N - 1, dim, generator=g)
    go = torch.randn(B, N, dim, generator=g)
    sd = ref.state_dict()
    for k in WEIGHT_NAMES:
        out[f"{tag}.{k}"] = sd[k].numpy()
    out[f"{tag}.x"] = x.numpy()
    out[f"{tag}.gy"] = gy.numpy()
    out[f"{tag}.go"] = go.numpy()
    out[f"{tag}.meta"] = np.array([B, N, H, Dh, R, seed, subsample], dtype=np.int64)
    ss = slice(None, None, subsample)

    xa = x.clone().requires_grad_()
    ya = y0.clone().requires_grad_()
    y1 = ref.cross_update_Y(xa, ya)
    y1.backward(gy)
    out[f"{tag}.y_new"] = y1.detach().numpy()[:, ss]
    out[f"{tag}.cuy_grad_x"] = xa.grad.numpy()[:, ss]
    out[f"{tag}.cuy_grad_y"] = ya.grad.numpy()[:, ss]
    for causal in (True, False):
        c = int(causal)
        xb = x.clone().requires_grad_()
        yb = y1.detach().clone().requires_grad_()
        mask = torch.ones(B, N) if causal else None
        o = ref(xb, xb, xb, y=yb, mask=mask)
        o.backward(go)
        out[f"{tag}.out_c{c}"] = o.detach().numpy()[:, ss]
        out[f"{tag}.fwd_grad_x_c{c}"] = xb.grad.numpy()[:, ss]
        out[f"{tag}.fwd_grad_y_c{c}"] = yb.grad.numpy()[:, ss]


def layers():
    out = {}
    layer_case("tiny", 2, 16, 3, 16, 2, 100, out)
    layer_case("small", 1, 64, 4, 32, 4, 200, out)
    layer_case("wide_window", 1, 32, 2, 8, 40, 300, out)      # radius larger than the sequence
    np.savez_compressed(os.path.join(HERE, "layer_eager.npz"), **out)
    # The fp32 layer case B2 H4 N512 Dh64 R16 (causal window 16): weights and inputs are stored in
    # full, so the tests do not depend on re-drawing them; of the outputs every 8th row is kept.
    out = {}
    layer_case("config1", 2, 512, 4, 64, 16, 0, out, subsample=8)
    np.savez_compressed(os.path.join(HERE, "layer_config1.npz"), **out)


def triton_ops():
    """Package ops under the Triton interpreter: the op-level API itself."""
    out = {}
    g = torch.Generator().manual_seed(7)
    # build_parent_nodes
    B, P, H, D = 2, 8, 3, 16
    names = ("Qp", "Kp", "Vp", "Kc", "Vc")
    ts = [torch.randn(B, P * (2 if n[1] == "c" else 1), H, D, generator=g).requires_grad_() for n in names]
    o = build_parent_nodes(*ts)
    go = torch.randn(o.shape, generator=g)
    o.backward(go)
    for n, t in zip(names, ts):
        out[f"parent.{n}"] = t.detach().numpy()
        out[f"parent.d{n}"] = t.grad.numpy()
    out["parent.out"] = o.detach().numpy()
    out["parent.go"] = go.numpy()
    # hierarchical_attention
    for tag, (B, N, H, D, R) in {"span_a": (2, 16, 3, 16, 2), "span_b": (1, 32, 2, 24, 5),
                                 "span_r0": (1, 16, 2, 16, 0)}.items():
        Q = torch.randn(B, N, H, D, generator=g)
        K = torch.randn(B, 2 * N - 1, H, D, generator=g)
        V = torch.randn(B, 2 * N - 1, H, D, generator=g)
        go = torch.randn(B, N, H, D, generator=g)
        out[f"{tag}.meta"] = np.array([B, N, H, D, R], dtype=np.int64)
        out[f"{tag}.Q"], out[f"{tag}.K"], out[f"{tag}.V"], out[f"{tag}.go"] = (
            Q.numpy(), K.numpy(), V.numpy(), go.numpy())
        for causal in (True, False):
            c = int(causal)
            t = build_tree_topology(N, is_causal=causal, device="cpu")
            q, k, v = (a.clone().requires_grad_() for a in (Q, K, V))
            o = hierarchical_attention(q, k, v, t["forward_idx"], t["backward_gather"],
                                       t["forward_mask"] if causal else None, R)
            o.backward(go)
            out[f"{tag}.out_c{c}"] = o.detach().numpy()
            out[f"{tag}.dQ_c{c}"] = q.grad.numpy()
            out[f"{tag}.dK_c{c}"] = k.grad.numpy()
            out[f"{tag}.dV_c{c}"] = v.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "triton_ops.npz"), **out)


def logits_ops():
    """(1) The softmax weights the package's forward saves (its `Weights` tensor, ops/functional.py:131-132),
    taken from the unmodified forward run by the Triton interpreter.  (2) The cross logits of the first prototype's
    build_hierarchical_logits (Hierarchical_Attention_Triton.py:414-454), its kernel launched as the prototype's
    own launcher does (:487-497); the prototype's self-logits kernel cannot be launched as shipped."""
    from hierarchical_attention.ops.functional import HierarchicalAttentionFunc

    class Ctx:
        def save_for_backward(self, *tensors):
            self.saved = tensors

    out = {}
    g = torch.Generator().manual_seed(17)
    for tag, (B, N, H, D, R) in {"w_a": (2, 16, 3, 16, 2), "w_b": (1, 32, 2, 8, 5), "w_r0": (1, 8, 2, 16, 0)}.items():
        Q = torch.randn(B, N, H, D, generator=g)
        K = torch.randn(B, 2 * N - 1, H, D, generator=g)
        V = torch.randn(B, 2 * N - 1, H, D, generator=g)
        out[f"{tag}.meta"] = np.array([B, N, H, D, R], dtype=np.int64)
        out[f"{tag}.Q"], out[f"{tag}.K"] = Q.numpy(), K.numpy()
        for causal in (True, False):
            t = build_tree_topology(N, is_causal=causal, device="cpu")
            ctx = Ctx()
            HierarchicalAttentionFunc.forward(ctx, Q, K, V, t["forward_idx"], t["backward_gather"],
                                              t["forward_mask"] if causal else None, R)
            out[f"{tag}.weights_c{int(causal)}"] = ctx.saved[5].numpy()
    spec = importlib.util.spec_from_file_location("ref_v1", os.path.join(REF, "Hierarchical_Attention_Triton.py"))
    v1 = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(v1)
    B, N, H, D = 2, 16, 4, 16                       # the prototype's kernels need a power-of-two head count
    total = 2 * N - 1
    Q = torch.randn(B, total, H * D, generator=g)
    K = torch.randn(B, total, H * D, generator=g)
    res = torch.empty(B, total - 1, H)
    v1.hierarchical_cross_logits_kernel_opt[(total - 1, B)](Q, K, res, *Q.stride(), *res.stride(), H=H, D=D,
                                                            BLOCK_SIZE_D=32, num_warps=4)
    out["v1.meta"] = np.array([B, N, H, D], dtype=np.int64)
    out["v1.ALL_Q"], out["v1.ALL_K"], out["v1.RES_CROSS"] = Q.numpy(), K.numpy(), res.numpy()
    np.savez_compressed(os.path.join(HERE, "logits_ops.npz"), **out)


if __name__ == "__main__":
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    topology()
    span_y()
    layers()
    triton_ops()
    logits_ops()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
