"""GPU side of the checkpoint reader: batched, double-buffered upload (bit-exact with the file) and an
EXL3 linear built from a weight set (markers select the codebook), checked against the oracle."""
import numpy as np
import pytest

from conftest import make_linear

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_upload_and_linear_from_a_checkpoint(tmp_path, oracle):
    from ampstein_b200 import models, weights
    k, n, K = 512, 384, 4
    tensors, lin = {}, {}
    for i, cbname in enumerate((None, "mul1", "mcg")):
        trellis, suh, svh, x = make_linear(k, n, K, seed=8800 + i, m=3)
        key = "model.layers.%d.mlp.down_proj" % i
        tensors[key + ".trellis"] = torch.from_numpy(trellis.view(np.int16).copy())
        tensors[key + ".suh"] = torch.from_numpy(suh.copy())
        tensors[key + ".svh"] = torch.from_numpy(svh.copy())
        if cbname:
            tensors[key + "." + cbname] = torch.zeros(1, dtype=torch.int32)
        if i == 1:
            tensors[key + ".bias"] = torch.randn(n).to(torch.bfloat16)
        lin[key] = (trellis, suh, svh, x, {None: 0, "mcg": 1, "mul1": 2}[cbname])
    tensors["big"] = torch.randint(-128, 127, (3, 1000, 333), dtype=torch.int8)          # odd sizes: offsets stay 256-aligned
    weights.save_file(tensors, str(tmp_path / "model.safetensors"))
    ws = weights.open(str(tmp_path))
    moved = ws.upload(0, batch_bytes=300 << 10)                                          # several batches through two staging buffers
    assert moved >= sum(t.numel() * t.element_size() for t in tensors.values())
    torch.cuda.synchronize()
    for key, t in tensors.items():
        g = ws.gpu(key)
        assert g.is_cuda and g.dtype == t.dtype and g.shape == t.shape and g.data_ptr() % 256 == 0
        assert torch.equal(g.cpu(), t)
    assert ws.upload(0) == 0                                                             # everything is cached
    for key, (trellis, suh, svh, x, cb) in lin.items():
        layer = models.linear(ws, key)
        assert (layer.mul1, layer.mcg) == (cb == 2, cb == 1) and layer.K == K
        y = layer.forward(torch.from_numpy(x).cuda()).float().cpu().numpy()
        ref = oracle.linear(x, trellis, suh, svh, cb, fp32_out=True)
        if layer.bias is not None:
            ref = ref + layer.bias.float().cpu().numpy()
        assert np.max(np.abs(y - ref)) / np.max(np.abs(ref)) < 1e-2
    # a tensor touched first through gpu() is uploaded on its own
    ws2 = weights.open(str(tmp_path))
    assert torch.equal(ws2.gpu("big").cpu(), tensors["big"])
