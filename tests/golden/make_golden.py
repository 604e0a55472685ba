"""Generates tests/golden/aten_golden.npz: small seeded input/output vectors from
PyTorch's CPU ATen kernels for the torch ops the reference's emitter targets
(include/fusilli/support/asm_emitter.h: aten.convolution :667-731,
aten.convolution_backward :856-903/:1018-1064, aten.matmul :1669-1696,
aten.scaled_dot_product_attention :2409-2468, aten.layer_norm /
native_layer_norm :1427-1503, aten.rms_norm :1592-1626, reductions
:2282-2317, pointwise table :1959-2116).

The reference itself (IREE llvm-cpu) cannot run on this machine, so these are
the closest executable statement of the semantics it lowers to. Run once:
    python tests/golden/make_golden.py
    python tests/golden/make_golden.py --batchnorm     (batchnorm_golden.npz, aten.native_batch_norm :1232-1307)
Inputs are float32 and computed in float64 so the vectors carry no
accumulation-order noise; tests compare the oracle to them at 1e-5.
"""
import os

import numpy as np
import torch
import torch.nn.functional as F

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "aten_golden.npz")


def main():
    torch.manual_seed(1234)
    g = {}
    d = torch.float64

    def rnd(*shape, lo=-1.0, hi=1.0):
        return (torch.rand(*shape, dtype=torch.float32) * (hi - lo) + lo)

    # ---- convolution: (name, N, C, H, W, K, R, S, pad, stride, dil, groups)
    conv_cases = [
        ("c3x3", 2, 8, 9, 10, 6, 3, 3, 1, 1, 1, 1),
        ("c1x1", 3, 16, 7, 7, 8, 1, 1, 0, 1, 1, 1),
        ("cgrp", 2, 8, 8, 8, 12, 3, 3, 1, 2, 1, 4),
        ("cdil", 1, 4, 11, 12, 5, 3, 2, 2, 1, 2, 1),
    ]
    for nm, N, C, H, W, K, R, S, p, s, dl, grp in conv_cases:
        x = rnd(N, C, H, W)
        w = rnd(K, C // grp, R, S)
        y = F.conv2d(x.to(d), w.to(d), None, s, p, dl, grp)
        dy = rnd(*y.shape)
        dx, dw, _ = torch.ops.aten.convolution_backward(
            dy.to(d), x.to(d), w.to(d), None, [s, s], [p, p], [dl, dl], False, [0, 0], grp,
            [True, True, False])
        g[f"conv_{nm}_meta"] = np.array([N, C, H, W, K, R, S, p, s, dl, grp])
        for k, v in (("x", x), ("w", w), ("y", y), ("dy", dy), ("dx", dx), ("dw", dw)):
            g[f"conv_{nm}_{k}"] = v.to(torch.float32).numpy()
    # 3-D convolution
    x = rnd(2, 4, 5, 6, 7)
    w = rnd(6, 4, 2, 3, 3)
    g["conv3d_x"], g["conv3d_w"] = x.numpy(), w.numpy()
    g["conv3d_y"] = F.conv3d(x.to(d), w.to(d), None, 1, (0, 1, 1)).to(torch.float32).numpy()

    # ---- matmul with batch broadcast
    a = rnd(4, 2, 9, 13)
    b = rnd(1, 2, 13, 7)
    g["mm_a"], g["mm_b"] = a.numpy(), b.numpy()
    g["mm_c"] = torch.matmul(a.to(d), b.to(d)).to(torch.float32).numpy()

    # ---- sdpa: plain, causal, additive mask, GQA
    q = rnd(2, 4, 10, 16)
    k = rnd(2, 4, 12, 16)
    v = rnd(2, 4, 12, 8)
    m = rnd(2, 1, 10, 12, lo=-2, hi=2)
    g["sdpa_q"], g["sdpa_k"], g["sdpa_v"], g["sdpa_mask"] = q.numpy(), k.numpy(), v.numpy(), m.numpy()
    g["sdpa_plain"] = F.scaled_dot_product_attention(q.to(d), k.to(d), v.to(d)).float().numpy()
    g["sdpa_causal"] = F.scaled_dot_product_attention(q.to(d), k.to(d), v.to(d), is_causal=True).float().numpy()
    g["sdpa_masked"] = F.scaled_dot_product_attention(q.to(d), k.to(d), v.to(d), attn_mask=m.to(d)).float().numpy()
    g["sdpa_scaled"] = F.scaled_dot_product_attention(q.to(d), k.to(d), v.to(d), scale=0.3).float().numpy()
    kg = rnd(2, 2, 12, 16)
    vg = rnd(2, 1, 12, 8)
    g["sdpa_kg"], g["sdpa_vg"] = kg.numpy(), vg.numpy()
    g["sdpa_gqa"] = F.scaled_dot_product_attention(
        q.to(d), kg.to(d).repeat_interleave(2, 1), vg.to(d).repeat_interleave(4, 1)).float().numpy()

    # ---- norms
    x = rnd(3, 5, 4, 6, lo=-2, hi=3)
    sc = rnd(1, 5, 4, 6)
    bi = rnd(1, 5, 4, 6)
    y, mean, rstd = torch.ops.aten.native_layer_norm(x.to(d), [5, 4, 6], sc[0].to(d), bi[0].to(d), 1e-5)
    g["ln_x"], g["ln_scale"], g["ln_bias"] = x.numpy(), sc.numpy(), bi.numpy()
    g["ln_y"], g["ln_mean"], g["ln_rstd"] = y.float().numpy(), mean.float().numpy(), rstd.float().numpy()
    g["rms_y"] = torch.ops.aten.rms_norm(x.to(d), [5, 4, 6], sc[0].to(d), 1e-5).float().numpy()

    # ---- reductions over dims (2,3) keepdim
    x = rnd(2, 6, 4, 5, lo=-1.5, hi=1.5)
    x[0, 0, 0, 0] = 0.0
    xd = x.to(d)
    g["red_x"] = x.numpy()
    dims = [2, 3]
    red = {
        "ADD": xd.sum(dims, keepdim=True), "MUL": torch.prod(torch.prod(xd, 3, True), 2, True),
        "MIN": xd.amin(dims, keepdim=True), "MAX": xd.amax(dims, keepdim=True),
        "AMAX": xd.abs().amax(dims, keepdim=True), "AVG": xd.mean(dims, keepdim=True),
        "NORM1": xd.abs().sum(dims, keepdim=True), "NORM2": (xd * xd).sum(dims, keepdim=True).sqrt(),
        "MUL_NO_ZEROS": torch.prod(torch.prod(torch.where(xd != 0, xd, torch.ones_like(xd)), 3, True), 2, True),
    }
    for kname, val in red.items():
        g[f"red_{kname}"] = val.float().numpy()

    # ---- pointwise
    a = rnd(3, 4, 5, lo=-3, hi=3)
    b = rnd(3, 4, 5, lo=-3, hi=3)
    ap = rnd(3, 4, 5, lo=0.1, hi=3)
    g["pw_a"], g["pw_b"], g["pw_ap"] = a.numpy(), b.numpy(), ap.numpy()
    A, B, AP = a.to(d), b.to(d), ap.to(d)
    un = {
        "ABS": A.abs(), "CEIL": A.ceil(), "FLOOR": A.floor(), "NEG": -A, "EXP": A.exp(),
        "ERF": A.erf(), "SIN": A.sin(), "TAN": A.tan(), "TANH_FWD": A.tanh(),
        "SIGMOID_FWD": A.sigmoid(), "RELU_FWD": A.relu(), "IDENTITY": A.clone(),
        "ELU_FWD": F.elu(A, 0.7), "GELU_FWD": F.gelu(A), "GELU_APPROX_TANH_FWD": F.gelu(A, approximate="tanh"),
        "SOFTPLUS_FWD": F.softplus(A, 1.5, 2.0), "SWISH_FWD": A * torch.sigmoid(1.3 * A),
    }
    unp = {"LOG": AP.log(), "SQRT": AP.sqrt(), "RSQRT": AP.rsqrt(), "RECIPROCAL": AP.reciprocal()}
    bi_ = {
        "ADD": A + B, "SUB": A - B, "MUL": A * B, "DIV": A / B, "MAX_OP": torch.maximum(A, B),
        "MIN_OP": torch.minimum(A, B), "ADD_SQUARE": A + B * B,
        "RELU_BWD": torch.ops.aten.threshold_backward(A, B, 0),
        "TANH_BWD": torch.ops.aten.tanh_backward(A, B.tanh()),
        "GELU_BWD": torch.ops.aten.gelu_backward(A, B, approximate="none"),
        "GELU_APPROX_TANH_BWD": torch.ops.aten.gelu_backward(A, B, approximate="tanh"),
        "SWISH_BWD": A * (torch.sigmoid(1.3 * B) + 1.3 * B * torch.sigmoid(1.3 * B) * (1 - torch.sigmoid(1.3 * B))),
    }
    for kname, val in un.items():
        g[f"pw1_{kname}"] = val.float().numpy()
    for kname, val in unp.items():
        g[f"pw1p_{kname}"] = val.float().numpy()
    for kname, val in bi_.items():
        g[f"pw2_{kname}"] = val.float().numpy()
    np.savez_compressed(OUT, **g)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(g), "arrays")


OUT_BN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "batchnorm_golden.npz")


def main_batchnorm():
    """tests/golden/batchnorm_golden.npz: aten.native_batch_norm, the op BatchNormNode lowers to
    (asm_emitter.h:1283-1284), in both phases, 4-D and 5-D, with and without the optional operands.
    A file and a seed of its own, so the vectors above stay byte-identical."""
    torch.manual_seed(4321)
    g = {}
    d = torch.float64
    for nm, shape in (("4d", (3, 5, 4, 6)), ("5d", (2, 3, 2, 3, 4)), ("2d", (7, 4))):
        c = shape[1]
        x = torch.rand(*shape, dtype=torch.float32) * 4 - 1
        w = torch.rand(c) + 0.5
        b = torch.rand(c) - 0.5
        rm = torch.rand(c) - 0.5
        rv = torch.rand(c) + 0.25
        g[f"bn_{nm}_x"], g[f"bn_{nm}_w"], g[f"bn_{nm}_b"] = x.numpy(), w.numpy(), b.numpy()
        g[f"bn_{nm}_rm"], g[f"bn_{nm}_rv"] = rm.numpy(), rv.numpy()
        y, _, _ = torch.ops.aten.native_batch_norm(x.to(d), w.to(d), b.to(d), rm.to(d), rv.to(d), False, 0.1, 1e-5)
        g[f"bn_{nm}_infer_y"] = y.float().numpy()
        y, sm, si = torch.ops.aten.native_batch_norm(x.to(d), w.to(d), b.to(d), None, None, True, 0.1, 1e-5)
        g[f"bn_{nm}_train_y"], g[f"bn_{nm}_train_mean"], g[f"bn_{nm}_train_invstd"] = (
            y.float().numpy(), sm.float().numpy(), si.float().numpy())
        y, sm, si = torch.ops.aten.native_batch_norm(x.to(d), None, None, None, None, True, 0.1, 1e-5)
        g[f"bn_{nm}_plain_y"] = y.float().numpy()
    np.savez_compressed(OUT_BN, **g)
    print("wrote", OUT_BN, os.path.getsize(OUT_BN), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    import sys
    if "--batchnorm" in sys.argv:
        main_batchnorm()
    else:
        main()
