"""Offline side of the WUSH block transform: solve T, transform the weights, and the fp64
statement of the activation transform.

Same three entry points and tensor conventions as the reference's
``my_int4/wush_transform.py:27-58``:

* ``compute_wush_transform(X_cal, W) -> T``  fp64, shape (K/32, 32, 32);
* ``transform_weights(W, T)``                 ``W' = W @ T^-1`` per 32-wide block;
* ``transform_activations_reference(X, T)``   ``X' = X @ T^T`` per block, so that
  ``X' W'^T == X W^T`` for every invertible T.

The reference delegates the solve to the external IST-DASLab/WUSH checkout
(``block_transform.get_wush_transform``), which is not part of the reference repository.  The
construction below is written from the published closed form (arXiv 2512.00956): with the
per-block second moments ``G_w = W_b^T W_b / N`` and ``G_x = X_b^T X_b / M``, Cholesky factors
``G_w = L_w L_w^T``, ``G_x = L_x L_x^T`` and the SVD ``L_w^T L_x = U S V^T``,

    T = H  S^(-1/2)  U^T  L_w^T

where H is the orthonormal 32x32 Hadamard matrix (identity when ``use_hadamard=False``).
with the singular values in ascending order.  Transformed activations ``T x`` and transformed
weights ``T^-T w`` then share the covariance ``H S H^T``: whitened, balanced between the two operands, and spread evenly over the 32
coordinates -- which is what makes a per-group 4-bit grid fit both sides.  No golden values
of T exist in the reference, so T itself is checked only through the reference's own gates
(product invariance in fp64 and the end-to-end error on outlier data).
"""
from __future__ import annotations

import torch


def hadamard(n: int, dtype=torch.float64, device=None) -> torch.Tensor:
    """Orthonormal Sylvester-Hadamard matrix; n must be a power of two."""
    assert n > 0 and n & (n - 1) == 0
    h = torch.ones(1, 1, dtype=dtype, device=device)
    while h.shape[0] < n:
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return h / (n ** 0.5)


def diag_block_gram(x: torch.Tensor, size: int = 32, dtype=torch.float64, rows_per_block: int = 8192) -> torch.Tensor:
    """(rows, K) -> (K/size, size, size): the diagonal blocks of x^T x, accumulated over row blocks so
    that only ``rows_per_block`` rows are ever widened to ``dtype`` at once (a 70B-size layer in fp64
    would be several GB otherwise)."""
    rows, K = x.shape
    assert K % size == 0
    gram = torch.zeros(K // size, size, size, dtype=dtype, device=x.device)
    for r0 in range(0, rows, rows_per_block):
        part = x[r0:r0 + rows_per_block]
        blocks = part.to(dtype).reshape(part.shape[0], K // size, size).permute(1, 0, 2)      # (C, rows, size)
        gram += blocks.transpose(1, 2) @ blocks
    return gram


def _chol(gram: torch.Tensor) -> torch.Tensor:
    """Lower Cholesky factor with a relative ridge that grows only if a block is singular."""
    eye = torch.eye(gram.shape[-1], dtype=gram.dtype, device=gram.device)
    level = gram.diagonal(dim1=-2, dim2=-1).mean(-1).clamp_min(1e-30)[:, None, None]
    ridge = 1e-10
    while True:
        factor, info = torch.linalg.cholesky_ex(gram + ridge * level * eye)
        if int(info.max()) == 0:
            return factor
        ridge *= 100.0
        if ridge > 1e-2:
            raise RuntimeError("diag-block Gram matrix is not positive definite")


def solve_from_grams(g_x: torch.Tensor, g_w: torch.Tensor, use_hadamard: bool = True) -> torch.Tensor:
    """Closed-form T from per-block second moments, both (K/G, G, G) fp64."""
    hi = torch.float64
    l_x, l_w = _chol(g_x.to(hi)), _chol(g_w.to(hi))
    u, s, _ = torch.linalg.svd(l_w.transpose(1, 2) @ l_x)
    # Ascending order: the first Hadamard column is constant, so whatever sits in coordinate 0
    # becomes a common offset of all 32 outputs.  The sigma-clip scale subtracts the group
    # mean, so a dominant direction placed there would be clipped (10.9 % instead of 7.8 %
    # end-to-end error on the reference's outlier recipe); the weakest direction is harmless.
    u, s = u.flip(-1), s.flip(-1)
    # A singular vector is defined up to its sign and LAPACK and cuSOLVER choose differently: make the
    # component of largest magnitude positive, so that the CPU and the GPU solve give the same T.
    pick = u.abs().argmax(dim=1, keepdim=True)                       # (C, 1, G): row of the largest entry per column
    u = u * torch.sign(torch.gather(u, 1, pick))
    t = (s.clamp_min(1e-300) ** -0.5).unsqueeze(-1) * (u.transpose(1, 2) @ l_w.transpose(1, 2))
    if use_hadamard:
        t = hadamard(t.shape[-1], hi, t.device) @ t
    return t


def compute_wush_transform(X_cal: torch.Tensor, W: torch.Tensor, group_size: int = 32,
                           use_hadamard: bool = True) -> torch.Tensor:
    """X_cal (M, K) calibration activations, W (N, K) weights -> T (K/G, G, G) fp64."""
    hi = torch.float64
    g_x = diag_block_gram(X_cal, group_size, hi) / X_cal.shape[0]
    g_w = diag_block_gram(W, group_size, hi) / W.shape[0]
    return solve_from_grams(g_x, g_w, use_hadamard)


def transform_weights(W: torch.Tensor, T: torch.Tensor) -> torch.Tensor:
    """W (N, K), T (K/G, G, G) -> W' = W @ T^-1 per block, fp64."""
    hi = torch.float64
    C, G, _ = T.shape
    wb = W.to(hi).reshape(W.shape[0], C, G).permute(1, 0, 2)                 # (C, N, G)
    # W'_b T_b = W_b   <=>   T_b^T W'_b^T = W_b^T
    out = torch.linalg.solve(T.to(hi).transpose(1, 2), wb.transpose(1, 2)).transpose(1, 2)
    return out.permute(1, 0, 2).reshape(W.shape[0], C * G)


def transform_activations_reference(X: torch.Tensor, T: torch.Tensor) -> torch.Tensor:
    """X (..., K), T (K/G, G, G) -> X' = X @ T^T per block, fp64."""
    hi = torch.float64
    C, G, _ = T.shape
    xb = X.to(hi).reshape(-1, C, G)
    out = torch.einsum("rci,cji->rcj", xb, T.to(hi))
    return out.reshape(*X.shape[:-1], C * G)
