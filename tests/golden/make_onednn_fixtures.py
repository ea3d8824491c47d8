"""Generates tests/golden/onednn_fixtures.npz: outputs of REAL oneDNN for the parts of the tensor hot
path that PyTorch's CPU build exposes through mkldnn tensors.

Run where PyTorch with oneDNN is installed:  python tests/golden/make_onednn_fixtures.py
The reference (Deep Diamond's DNNL backend) calls the same oneDNN primitives through JavaCPP
(eltwise forward: dnnl/impl.clj:324-331; reorder: :372-376; sum: :345-359; binary: :363-368); the
oneDNN bundled with PyTorch is a different release from the one the reference pins (3.13), which
the fixture records.  What PyTorch does not expose through mkldnn tensors (elu, the other kinds of the
reference's eltwise table apart from gelu-erf, eltwise backward,
broadcast binary, reductions, plain nhwc reorders, int8) has no fixture here.
"""
import os

import numpy as np
import torch

N = 2048


def main():
    out = {}
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(N) * 2.0).astype(np.float32)
    x[:8] = [0.0, -0.0, 1.0, -1.0, 10.0, -10.0, 30.0, -30.0]
    tx = torch.from_numpy(x).reshape(1, N, 1, 1).to_mkldnn()
    out["x"] = x
    out["relu"] = torch.relu(tx).to_dense().numpy().reshape(-1)
    out["logistic"] = torch.sigmoid(tx).to_dense().numpy().reshape(-1)
    out["tanh"] = torch.tanh(tx).to_dense().numpy().reshape(-1)
    out["gelu_erf"] = torch.nn.functional.gelu(tx).to_dense().numpy().reshape(-1)  # eltwise_gelu_erf

    rng = np.random.default_rng(6)
    c = rng.standard_normal(N).astype(np.float32)
    c[:4] = [1.0, 1.00390625, 1.01171875, -3.0]  # exact, tie-to-even down, tie-to-even up, exact
    tb = torch.from_numpy(c).reshape(1, N, 1, 1).to_mkldnn(torch.bfloat16).to_dense()
    out["cvt_in"] = c
    out["cvt_bf16_bits"] = tb.view(torch.int16).numpy().reshape(-1).view(np.uint16)

    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, N).astype(np.float32)
    b = rng.uniform(0.5, 1.5, N).astype(np.float32)
    ta = torch.from_numpy(a).reshape(1, N, 1, 1).to_mkldnn()
    tb2 = torch.from_numpy(b).reshape(1, N, 1, 1).to_mkldnn()
    out["a"], out["b"] = a, b
    out["add"] = (ta + tb2).to_dense().numpy().reshape(-1)
    out["mul"] = (ta * tb2).to_dense().numpy().reshape(-1)

    cfg = torch.__config__.show()
    ver = [ln.strip(" -") for ln in cfg.splitlines() if "MKL-DNN" in ln or "oneDNN" in ln]
    out["onednn_version"] = np.array(ver[0] if ver else "unknown")
    out["torch_version"] = np.array(torch.__version__)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "onednn_fixtures.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, "|", out["onednn_version"])


if __name__ == "__main__":
    main()
