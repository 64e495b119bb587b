"""numpy restatement of the reference's MLP predictor forward -- TEST INFRASTRUCTURE ONLY.

Follows RuntimePredictor.predict (analyzer/habitat/analysis/mlp/mlp.py:252-267)
applied to a whole [Q, F+4] matrix at once: float64 normalisation
(mlp.py:258-261), cast to float32 (mlp.py:264), then fc1 + ReLU, the hidden
Linear + ReLU stack and fc2 (mlp.py:17-50) in float32 (or float64 as a
tie-breaker).  The arithmetic itself is torch's CPU nn.Linear in the reference
(torch is pinned at 1.4.0 there, docker/Dockerfile:14); a BLAS sgemm here.
Pinned against the reference's own predict() by tests/golden fixtures.
"""
import numpy as np


def normalise(op_features, device_rows, device_features, mu, sigma):
    x = np.concatenate([np.asarray(op_features, dtype=np.float64),
                        np.asarray(device_features, dtype=np.float64)[np.asarray(device_rows)]],
                       axis=1)
    return (x - np.asarray(mu, np.float64)) / np.asarray(sigma, np.float64)


def forward(weights, x_norm, dtype=np.float32, return_layers=False):
    """weights: dict(fc1_w, fc1_b, hidden_w [L, W, W], hidden_b [L, W], fc2_w [W], fc2_b [1])."""
    h = np.asarray(x_norm).astype(np.float32).astype(dtype)   # the reference casts to float32 first
    acts = []
    h = np.maximum(h @ weights["fc1_w"].astype(dtype).T + weights["fc1_b"].astype(dtype), 0)
    acts.append(h)
    for L in range(weights["hidden_w"].shape[0]):
        h = np.maximum(h @ weights["hidden_w"][L].astype(dtype).T + weights["hidden_b"][L].astype(dtype), 0)
        acts.append(h)
    out = h @ weights["fc2_w"].astype(dtype).reshape(-1) + weights["fc2_b"].astype(dtype).reshape(-1)[0]
    return (out, acts) if return_layers else out


def predict(weights, op_features, device_rows, device_features, mu, sigma, dtype=np.float32,
            chunk=16384):
    outs = []
    n = len(op_features)
    for i in range(0, n, chunk):
        xn = normalise(op_features[i:i + chunk], device_rows[i:i + chunk], device_features, mu, sigma)
        outs.append(forward(weights, xn, dtype))
    return np.concatenate(outs) if outs else np.zeros((0,), dtype)


def bf16_round(x):
    """float32 values rounded to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + (((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF))) & np.uint32(0xFFFF0000)
    return r.view(np.float32)


def forward_bf16(weights, x_norm, depth=None):
    """The arithmetic of the device's bf16 mode, replayed in numpy: where the kernel rounds to
    bfloat16 (hidden-layer weights and activations) this rounds too, everything else is float32.
    fc1 keeps x and w as bf16 hi + lo parts and adds the products hi.hi + lo.hi + hi.lo; fc2 works on
    the unrounded float32 activations of the last hidden layer.  The only difference left to the
    device is the order of the float32 additions inside a dot product.  Not part of the reference:
    it pins the kernel far more tightly than a comparison with the float64 forward can."""
    x = np.asarray(x_norm).astype(np.float32)
    w1 = weights["fc1_w"].astype(np.float32)
    xh, wh = bf16_round(x), bf16_round(w1)
    xl, wl = bf16_round(x - xh), bf16_round(w1 - wh)
    z = (xh @ wh.T + xl @ wh.T + xh @ wl.T).astype(np.float32) + weights["fc1_b"].astype(np.float32)
    h = np.maximum(z, 0)
    n_hidden = weights["hidden_w"].shape[0] if depth is None else depth
    for L in range(n_hidden):
        a = bf16_round(h)
        w = bf16_round(weights["hidden_w"][L].astype(np.float32))
        h = np.maximum((a @ w.T).astype(np.float32) + weights["hidden_b"][L].astype(np.float32), 0)
    return (h @ weights["fc2_w"].astype(np.float32).reshape(-1) +
            weights["fc2_b"].astype(np.float32).reshape(-1)[0]).astype(np.float32)
