"""Generates tests/golden/lm_ops_golden.npz from PyTorch CPU ops (fp32).

The reference ships no golden vectors and its native modules cannot be built against this
PyTorch / CUDA, so the fixtures come from the PyTorch ops each low-memory operator replaces,
plus numpy restatements of the packed formats written independently of oracle/ (plain loops).
Run from the repository root:  python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "lm_ops_golden.npz"


def pack_bits_loop(flags):
    out = np.zeros((len(flags) + 7) // 8, dtype=np.uint8)
    for i, f in enumerate(flags):
        if f:
            out[i // 8] |= 1 << (7 - i % 8)
    return out


def pack_nibbles_loop(v):
    out = np.zeros((len(v) + 1) // 2, dtype=np.uint8)
    for i, x in enumerate(v):
        out[i // 2] |= (int(x) & 15) << (4 if i % 2 == 0 else 0)
    return out


def main():
    g = torch.Generator().manual_seed(1234)
    d = {}
    x = torch.randn(1003, generator=g)
    x[5] = 0.0
    d["relu_x"] = x.numpy()
    d["relu_mask"] = pack_bits_loop((x > 0).numpy())
    nib = torch.randint(0, 16, (77,), generator=g).numpy().astype(np.uint8)
    d["nib_in"], d["nib_out"] = nib, pack_nibbles_loop(nib)

    px = torch.randn(2, 3, 9, 11, generator=g)
    y, gi = F.max_pool2d(px, 3, 2, 1, return_indices=True)
    W = px.shape[3]
    local = np.zeros(gi.shape, dtype=np.uint8)
    for n in range(gi.shape[0]):
        for c in range(gi.shape[1]):
            for p in range(gi.shape[2]):
                for q in range(gi.shape[3]):
                    h, w = divmod(int(gi[n, c, p, q]), W)
                    local[n, c, p, q] = (h - (p * 2 - 1)) * 3 + (w - (q * 2 - 1))
    dy = torch.randn(y.shape, generator=g)
    pr = px.clone().requires_grad_(True)
    F.max_pool2d(pr, 3, 2, 1).backward(dy)
    d.update(pool_x=px.numpy(), pool_y=y.numpy(), pool_local=local,
             pool_nibbles=pack_nibbles_loop(local.reshape(-1)), pool_dy=dy.numpy(), pool_dx=pr.grad.numpy())

    bx = torch.randn(3, 5, 4, 6, generator=g) * 2 + 1
    gamma = torch.rand(5, generator=g) + 0.5
    beta = torch.randn(5, generator=g)
    bdy = torch.randn(bx.shape, generator=g)
    xr, gr, br = bx.clone().requires_grad_(True), gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    by = F.batch_norm(xr, None, None, gr, br, True, 0.1, 1e-5)
    by.backward(bdy)
    mean = bx.double().mean((0, 2, 3))
    var = bx.double().var((0, 2, 3), unbiased=False)
    d.update(bn_x=bx.numpy(), bn_gamma=gamma.numpy(), bn_beta=beta.numpy(), bn_y=by.detach().numpy(),
             bn_mean=mean.float().numpy(), bn_invstd=(1 / torch.sqrt(var + 1e-5)).float().numpy(),
             bn_dy=bdy.numpy(), bn_dx=xr.grad.numpy(), bn_dgamma=gr.grad.numpy(), bn_dbeta=br.grad.numpy())

    logits = torch.randn(4, 7, generator=g).requires_grad_(True)
    labels = torch.randint(0, 7, (4,), generator=g)
    loss = F.cross_entropy(logits, labels, reduction="none")
    loss.sum().backward()
    d.update(ce_logits=logits.detach().numpy(), ce_labels=labels.numpy(), ce_loss=loss.detach().numpy(),
             ce_dlogits=(logits.grad * 0.25).numpy())

    # the stem of the CPU-runnable configuration at a reduced size (1 x 3 x 32 x 32), same seeds
    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    gs = torch.Generator().manual_seed(0)
    sx = torch.randn(1, 3, 32, 32, generator=gs)
    sw = torch.empty(64, 3, 7, 7).normal_(0.0, (2.0 / (64 * 49)) ** 0.5, generator=gs)
    sdy = torch.randn(1, 64, 8, 8, generator=gs)
    wr = sw.clone().requires_grad_(True)
    c = F.conv2d(sx, wr, None, 2, 3)
    b = F.batch_norm(c, None, None, torch.ones(64), torch.zeros(64), True, 0.1, 1e-5)
    r = torch.relu(b)
    sy, sgi = F.max_pool2d(r, 3, 2, 1, return_indices=True)
    sy.backward(sdy)
    slocal = np.zeros(sgi.shape, dtype=np.uint8)
    for ch in range(64):
        for p in range(8):
            for q in range(8):
                h, w = divmod(int(sgi[0, ch, p, q]), 16)
                slocal[0, ch, p, q] = (h - (p * 2 - 1)) * 3 + (w - (q * 2 - 1))
    d.update(stem_y=sy.detach().numpy(), stem_mask=pack_bits_loop((b.detach().reshape(-1) > 0).numpy()),
             stem_nibbles=pack_nibbles_loop(slocal.reshape(-1)), stem_dw=wr.grad.numpy())
    np.savez_compressed(OUT, **d)
    print("wrote", OUT, {k: v.shape for k, v in d.items()})


if __name__ == "__main__":
    main()
