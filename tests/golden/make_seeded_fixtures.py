"""Writes seeded_fixtures.npz: seeded inputs of the hot-path operators at small tensor-core-eligible sizes and the
outputs the f64-accumulating CPU oracle computes for them.  The GPU parity tests compare the device against these
files (the oracle need not be built where they run); the CPU tests check that the oracle still reproduces them.
Run from the repository root:  python tests/golden/make_seeded_fixtures.py"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def build():
    from oracle.nrs_oracle import Oracle
    o = Oracle("f64")
    rng = np.random.default_rng(20240607)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    out = {}
    # convolution 32 -> 32 channels, 3x3 s1 p1 on 2 images of 8x8 (one 128-pixel tile)
    x, w, b = f(2, 32, 8, 8), (f(32, 32, 3, 3) * 0.06).astype(np.float32), f(32) * 0.1
    dy = f(2, 32, 8, 8)
    dx, dw, db = o.conv2d_bwd(x, w, dy, 1, 1)
    out.update(conv_x=x, conv_w=w, conv_b=b, conv_dy=dy, conv_y=o.conv2d_fwd(x, w, b, 1, 1), conv_dx=dx, conv_dw=dw, conv_db=db)
    # matmul 32 x 64 x 32 and its two gradients
    a, bm, dc = f(32, 64), f(64, 32), f(32, 32)
    da, dbm = o.matmul_bwd(a, bm, dc)
    out.update(mm_a=a, mm_b=bm, mm_dc=dc, mm_c=o.matmul_fwd(a, bm), mm_da=da, mm_db=dbm)
    # layernorm over 8 rows of 64
    lx, lg, lb, lgy = f(8, 64) * 2 + 0.5, f(64) * 0.5 + 1, f(64) * 0.1, f(8, 64)
    ly, lxhat, listd = o.layernorm_fwd(lx, lg, lb, 1e-5)
    ldx, ldg, ldb = o.layernorm_bwd(lgy, lxhat, listd, lg)
    out.update(ln_x=lx, ln_gamma=lg, ln_beta=lb, ln_gy=lgy, ln_y=ly, ln_xhat=lxhat, ln_istd=listd, ln_dx=ldx, ln_dgamma=ldg,
               ln_dbeta=ldb)
    # softmax over 8 rows of 128
    sx, sg = f(8, 128) * 3, f(8, 128)
    sy = o.softmax_fwd(sx)
    out.update(sm_x=sx, sm_g=sg, sm_y=sy, sm_dx=o.softmax_bwd(sy, sg))
    # cross-entropy, 16 rows of 20 classes, one-hot targets
    cl, ct = f(16, 20) * 2, np.eye(20, dtype=np.float32)[rng.integers(0, 20, 16)]
    out.update(ce_logits=cl, ce_target=ct, ce_loss=np.float32(o.ce_fwd(cl, ct)), ce_grad=o.ce_bwd(cl, ct))
    # max-pool 2x2 on [2, 4, 8, 8] (distinct values: no ties)
    px = rng.permutation(2 * 4 * 8 * 8).astype(np.float32).reshape(2, 4, 8, 8) * 0.01
    py, pam = o.maxpool_fwd(px, 2, 2)
    pg = f(*py.shape)
    out.update(pool_x=px, pool_y=py, pool_argmax=pam, pool_gy=pg, pool_dx=o.maxpool_bwd(pg, pam, px.shape))
    # GELU
    gx, gg = f(256) * 2, f(256)
    out.update(gelu_x=gx, gelu_g=gg, gelu_y=o.gelu_fwd(gx), gelu_dx=o.gelu_bwd(gx, gg))
    # AdamW: three steps with fresh gradients
    p, m, v = f(200), np.zeros(200, np.float32), np.zeros(200, np.float32)
    grads = f(3, 200)
    out.update(adamw_p0=p.copy(), adamw_grads=grads)
    for t in range(3):
        o.adamw_step(p, grads[t], m, v, 1e-3, 0.9, 0.999, 1e-8, 1e-4, t)
    out.update(adamw_p3=p, adamw_m3=m, adamw_v3=v)
    return out


if __name__ == "__main__":
    np.savez_compressed(Path(__file__).parent / "seeded_fixtures.npz", **build())
    print("wrote", Path(__file__).parent / "seeded_fixtures.npz")
