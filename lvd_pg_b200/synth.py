"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (there is no ImageNet32/64 or MNIST on the machines this runs on; these
generators stand in for them).

  config 1  tree-structured Bernoulli data over 64 binary variables, HCLT k=16 on its Chow-Liu tree
  config 2  32x32x3 blurred-noise uint8 images (3072 variables, 256 categories), HCLT k=32
  config 3  64x64x3 images cut into 64 patches of 8x8x3 (192 variables each), HCLT k=128 per patch
  config 4  HCLT k=64 over 784 binary variables on a random spanning tree (KLD / sampling)
  config 5  config 2's data, HCLT k=256
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import structures as st


def tree_bernoulli_data(rows: int, v: int, seed: int) -> np.ndarray:
    """Ancestral samples of a random tree-structured Bernoulli model: random spanning tree, root
    marginal and every conditional P(x_child = 1 | x_parent) ~ U(0.1, 0.9)."""
    rng = np.random.default_rng(seed)
    parent = st.root_tree_at_center(v, st.random_spanning_tree(v, rng))
    order = [int(np.nonzero(parent < 0)[0][0])]
    ch = [[] for _ in range(v)]
    for x, p in enumerate(parent):
        if p >= 0:
            ch[int(p)].append(x)
    for u in order:
        order.extend(ch[u])
    cond = rng.uniform(0.1, 0.9, (v, 2))
    data = np.zeros((rows, v), np.uint8)
    for x in order:
        if parent[x] < 0:
            p1 = np.full(rows, cond[x, 0])
        else:
            p1 = cond[x, data[:, parent[x]]]
        data[:, x] = rng.random(rows) < p1
    return data


def blurred_noise_images(rows: int, side: int, sigma: float, seed: int, device="cpu", chunk: int = 4096) -> torch.Tensor:
    """uint8 images [rows, side*side*3]: Gaussian noise fields blurred spatially (sigma px),
    correlated 0.8 across channels (each channel mixes a shared field with its own), scaled to
    mean 128 / std 50, rounded and clipped to [0, 255].  Variable order is (y, x, channel)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    rad = max(1, int(3 * sigma))
    xs = torch.arange(-rad, rad + 1, dtype=torch.float32, device=dev)
    ker = torch.exp(-0.5 * (xs / sigma) ** 2)
    ker = ker / ker.sum()
    out = torch.empty(rows, side * side * 3, dtype=torch.uint8, device=dev)
    for r0 in range(0, rows, chunk):
        n = min(chunk, rows - r0)
        z = torch.randn(n, 4, side, side, generator=gen, device=dev)
        z = z.reshape(n * 4, 1, side, side)
        z = torch.nn.functional.conv2d(torch.nn.functional.pad(z, (rad, rad, 0, 0), mode="circular"), ker.view(1, 1, 1, -1))
        z = torch.nn.functional.conv2d(torch.nn.functional.pad(z, (0, 0, rad, rad), mode="circular"), ker.view(1, 1, -1, 1))
        z = z.reshape(n, 4, side, side)
        z = z / z.std()
        img = (0.8 ** 0.5) * z[:, :1] + (0.2 ** 0.5) * z[:, 1:]      # [n, 3, side, side]
        img = (img * 50.0 + 128.0).round().clamp(0, 255).to(torch.uint8)
        out[r0:r0 + n] = img.permute(0, 2, 3, 1).reshape(n, -1)
    return out


def image_clt(images: torch.Tensor, rows: int = 4096, bins: int = 32) -> np.ndarray:
    """Chow-Liu tree of image variables.  The pairwise mutual information is estimated on the
    first `rows` images with pixel values quantised to `bins` levels (structure learning is
    set-up, not part of the timed path; only the tree topology is used)."""
    sub = images[:rows]
    q = (sub.to(torch.int64) * bins // 256).to(torch.uint8)
    dev = "cuda" if q.is_cuda else "cpu"
    mi = st.pairwise_mi(q.cpu().numpy(), bins, 0.1, device=dev, chunk=128)
    np.fill_diagonal(mi, -np.inf)
    return st.root_tree_at_center(mi.shape[0], st.max_spanning_tree(mi))


def config1(seed: int = 1):
    data = tree_bernoulli_data(10000, 64, seed)
    parent = st.learn_clt(data, 2, 0.1)
    fc = st.hclt_flat(parent, 2, 16, seed=seed + 1)
    return data, fc


def config4(seed: int = 4, v: int = 784, k: int = 64):
    rng = np.random.default_rng(seed)
    parent = st.root_tree_at_center(v, st.random_spanning_tree(v, rng))
    q = st.hclt_flat(parent, 2, k, seed=seed * 10 + 1)
    p = st.hclt_flat(parent, 2, k, seed=seed * 10 + 2)
    return q, p


def image_hclt(k: int, rows: int, side: int = 32, sigma: float = 2.0, seed: int = 3, device="cpu",
               clt_rows: int = 4096, num_vars: Optional[int] = None):
    """Data and HCLT of configs 2 and 5 (side=32) — `num_vars` truncates to the first variables
    for reduced-size test cases."""
    images = blurred_noise_images(rows, side, sigma, seed, device)
    if num_vars is not None:
        images = images[:, :num_vars].contiguous()
    parent = image_clt(images, clt_rows)
    fc = st.hclt_flat(parent, 256, k, seed=seed + 1)
    return images, fc


def config3(rows: int = 20000, k: int = 128, seed: int = 3, device="cpu", patches: int = 64):
    """Config 3: 64x64x3 images (sigma = 4 px) cut into 64 non-overlapping 8x8x3 patches of 192
    variables; one HCLT (k latents, 256 categories) per patch position.  Returns a list of
    (patch data [rows, 192] uint8, FlatCircuit)."""
    images = blurred_noise_images(rows, 64, 4.0, seed, device)
    img = images.view(rows, 64, 64, 3)
    out = []
    for p in range(patches):
        py, px = divmod(p, 8)
        data = img[:, 8 * py:8 * py + 8, 8 * px:8 * px + 8, :].reshape(rows, 192).contiguous()
        parent = image_clt(data, 4096)
        out.append((data, st.hclt_flat(parent, 256, k, seed=seed + 1 + p)))
    return out
