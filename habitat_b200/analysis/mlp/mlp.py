"""MLP runtime predictors: the reference's load / save / predict API on the B200 kernel.

Reference: analyzer/habitat/analysis/mlp/mlp.py.  The torch modules keep the
reference's attribute names (fc1, mlp.layers.{0,2,...}, fc2, features) so its
checkpoints ({"mu", "sigma", "model": state_dict}, mlp.py:133-146) load
unchanged.  The modules only hold parameters: inference runs in the fused
sm_100a kernel (habitat_b200/csrc/mlp_chain.cu) through `predict_batch`, and
`predict` is that path with one query.  Training is out of scope.
"""
import numpy as np
import torch
import torch.nn as nn

from habitat_b200.analysis.mlp.devices import get_all_devices, get_device_features

FEATURES = {
    "linear": ["bias", "batch", "in_features", "out_features"],
    "lstm": ["bias", "bidirectional", "batch", "seq_len", "input_size", "hidden_size",
             "num_layers"],
    "conv2d": ["bias", "batch", "image_size", "in_channels", "out_channels", "kernel_size",
               "stride", "padding"],
    "bmm": ["batch", "left", "middle", "right"],
}


class MLPBase(nn.Module):
    """`layers` x [Linear(layer_size, layer_size), ReLU] (mlp.py:17-31)."""

    def __init__(self, layers, layer_size):
        super().__init__()
        blocks = []
        for _ in range(layers):
            blocks += [nn.Linear(layer_size, layer_size), nn.ReLU()]
        self.layers = nn.ModuleList(blocks)

    def forward(self, x):
        for block in self.layers:
            x = block(x)
        return x


class _OpMLP(nn.Module):
    """fc1 (F + 4 -> layer_size) + ReLU, MLPBase, fc2 (layer_size -> 1); mlp.py:34-109."""

    op_name = None

    def __init__(self, layers, layer_size):
        super().__init__()
        self.features = list(FEATURES[self.op_name])
        self.fc1 = nn.Linear(len(self.features) + 4, layer_size)
        self.mlp = MLPBase(layers, layer_size)
        self.fc2 = nn.Linear(layer_size, 1)

    def forward(self, x):
        return self.fc2(self.mlp(torch.relu(self.fc1(x))))


class LinearMLP(_OpMLP):
    op_name = "linear"


class LSTMMLP(_OpMLP):
    op_name = "lstm"


class Conv2DMLP(_OpMLP):
    op_name = "conv2d"


class BMMMLP(_OpMLP):
    op_name = "bmm"


_MODEL_CLASSES = {"linear": LinearMLP, "lstm": LSTMMLP, "conv2d": Conv2DMLP, "bmm": BMMMLP}


def state_to_arrays(model):
    """Weights of an _OpMLP as the numpy arrays the native library packs."""
    sd = {k: v.detach().cpu().float().numpy() for k, v in model.state_dict().items()}
    n_hidden = len(model.mlp.layers) // 2
    return dict(
        fc1_w=sd["fc1.weight"], fc1_b=sd["fc1.bias"],
        hidden_w=np.stack([sd["mlp.layers.%d.weight" % (2 * i)] for i in range(n_hidden)]),
        hidden_b=np.stack([sd["mlp.layers.%d.bias" % (2 * i)] for i in range(n_hidden)]),
        fc2_w=sd["fc2.weight"].reshape(-1), fc2_b=sd["fc2.bias"].reshape(-1))


class RuntimePredictor:
    """mlp.py:112-146, 252-267: same constructor, attributes and predict()."""

    def __init__(self, model_name, layers, layer_size, model_path=None, precision="bf16"):
        self.model_name = model_name
        self.layers = layers
        self.layer_size = layer_size
        self.model = _MODEL_CLASSES[model_name](layers, layer_size)
        self.device_params = ["mem", "mem_bw", "num_sm", "single"]
        self.mu = None
        self.sigma = None
        self.precision = precision
        self._handle = None
        self._device_rows = None
        if model_path is not None:
            self.load_state(model_path)

    # -- checkpoints --------------------------------------------------------
    def load_state(self, path):
        # mu / sigma are numpy arrays inside the checkpoint, which torch >= 2.6
        # only unpickles with weights_only=False
        checkpoint = torch.load(path, map_location="cpu", weights_only=False)
        self.mu = checkpoint["mu"]
        self.sigma = checkpoint["sigma"]
        self.model.load_state_dict(checkpoint["model"])
        self.invalidate()

    def save_state(self, path):
        torch.save({"mu": self.mu, "sigma": self.sigma, "model": self.model.state_dict()}, path)

    def invalidate(self):
        """Drops the device-side weight pack (call after changing weights, mu or sigma)."""
        if self._handle is not None:
            self._handle.close()
        self._handle = None
        self._device_rows = None

    # -- inference ----------------------------------------------------------
    def _ensure_handle(self):
        if self._handle is not None:
            return
        from habitat_b200.batched import MLPHandle
        if self.mu is None or self.sigma is None:
            raise RuntimeError("RuntimePredictor has no mu/sigma (load a checkpoint first)")
        devices = get_all_devices(self.device_params)
        names = sorted(devices)
        self._device_rows = {name: i for i, name in enumerate(names)}
        table = np.array([devices[n] for n in names], dtype=np.float64)
        arrays = state_to_arrays(self.model)
        self._handle = MLPHandle(len(self.model.features), mu=np.asarray(self.mu, np.float64),
                                 sigma=np.asarray(self.sigma, np.float64), device_features=table,
                                 precision=self.precision, **arrays)

    def device_row(self, device_name):
        self._ensure_handle()
        if device_name not in self._device_rows:
            get_device_features(device_name, self.device_params)  # raises like the reference
            self.invalidate()
            self._ensure_handle()
        return self._device_rows[device_name]

    def predict_batch(self, op_features, device_rows):
        """op_features [Q, F] float32 CUDA tensor, device_rows [Q] uint8 CUDA tensor
        (indices from device_row()).  Returns [Q] float32 predictions (ms), on the
        current stream, unsynchronised."""
        self._ensure_handle()
        return self._handle.predict(op_features, device_rows)

    def predict(self, kernel_arguments, device_name):
        """One query; same arguments and return type as the reference."""
        row = self.device_row(device_name)
        feats = torch.tensor([list(kernel_arguments)], dtype=torch.float32, device="cuda")
        rows = torch.tensor([row], dtype=torch.uint8, device="cuda")
        out = self._handle.predict(feats, rows)
        value = float(out.cpu()[0])
        self._handle.check_status()
        return value
