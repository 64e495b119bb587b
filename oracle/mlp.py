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
