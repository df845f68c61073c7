"""The saved {wq, ws, T} layer format: round trip, refusal of damaged or foreign files, and that
the offline pipeline gives the same file whether it runs blockwise or in one piece (CPU); on a GPU,
that the device pipeline reproduces the CPU pipeline's codes and scales bit for bit."""
import numpy as np
import pytest
import torch


def _small_layer(seed=0, K=256, N=96, rows_per_block=8192):
    from wush_int4_kernel_b200 import layer_file, synth

    gen = torch.Generator().manual_seed(seed)
    outliers = synth.outlier_channels(K, gen)
    x_cal = synth.draw_activations(64, K, outliers, gen).float()
    W = (0.02 * torch.randn(N, K, generator=gen)).to(torch.bfloat16)
    return W, x_cal, layer_file.prepare_layer(W, x_cal, rows_per_block=rows_per_block)


def test_round_trip_and_header(tmp_path):
    from wush_int4_kernel_b200 import layer_file

    W, x_cal, (wq, ws, t, t64) = _small_layer()
    path = str(tmp_path / "layer.pt")
    layer_file.save_layer(path, wq, ws, t, meta={"seed": 0, "source": "unit test"})
    back = layer_file.load_layer(path)
    assert (back.K, back.N) == (256, 96)
    assert torch.equal(back.wq, wq) and torch.equal(back.ws.view(torch.int16), ws.view(torch.int16))
    assert torch.equal(back.t_bf16.view(torch.int16), t.view(torch.int16))
    assert back.meta == {"seed": 0, "source": "unit test"}
    doc = torch.load(path, weights_only=True)                       # plain tensors and values only
    assert doc["format"] == "wush-w4a4-layer" and doc["version"] == 1 and doc["group_size"] == 32
    assert abs(doc["clip_sigmas"] - 2.473650) < 1e-12


def test_blockwise_pipeline_is_identical():
    _, _, (wq, ws, t, _) = _small_layer(seed=3)
    _, _, (wq_b, ws_b, t_b, _) = _small_layer(seed=3, rows_per_block=40)     # 96 rows in blocks of 40, 40, 16
    assert torch.equal(wq, wq_b) and torch.equal(ws.view(torch.int16), ws_b.view(torch.int16))
    assert torch.equal(t.view(torch.int16), t_b.view(torch.int16))


def test_quantised_layer_reproduces_the_product(orc):
    """What the file holds is what the path consumes: X' W'^T from the stored triple agrees with the
    unquantised X W^T to the accuracy INT4 allows on outlier-free data."""
    from wush_int4_kernel_b200 import wush_transform as wt

    W, x_cal, (wq, ws, t, t64) = _small_layer(seed=5, K=512, N=64)
    x = x_cal[:16].to(torch.bfloat16)
    xq, xs = orc.fused_tq(orc.bits(x), orc.bits(t))
    y = orc.gemm_f64(xq, xs, wq.numpy(), orc.bits(ws))
    y_true = (x.double() @ W.double().t()).numpy()
    assert np.linalg.norm(y - y_true) / np.linalg.norm(y_true) < 0.2
    # the fp64 transform pair leaves the product unchanged (the reference's invariance gate)
    inv = wt.transform_activations_reference(x.double(), t64) @ wt.transform_weights(W.double(), t64).t()
    assert np.linalg.norm(inv.numpy() - y_true) / np.linalg.norm(y_true) < 1e-9


def test_refuses_damaged_and_foreign_files(tmp_path):
    from wush_int4_kernel_b200 import layer_file

    _, _, (wq, ws, t, _) = _small_layer()
    path = str(tmp_path / "layer.pt")
    layer_file.save_layer(path, wq, ws, t)
    doc = torch.load(path, weights_only=True)
    bad = dict(doc)
    bad["wq"] = doc["wq"].clone()
    bad["wq"][0, 0] ^= 1
    torch.save(bad, path)
    with pytest.raises(ValueError, match="checksum"):
        layer_file.load_layer(path)
    assert layer_file.load_layer(path, verify=False).N == 96
    torch.save(dict(doc, version=2), path)
    with pytest.raises(ValueError, match="version"):
        layer_file.load_layer(path)
    torch.save({"format": "something else"}, path)
    with pytest.raises(ValueError, match="not a"):
        layer_file.load_layer(path)
    torch.save(dict(doc, ws=doc["ws"][:, :-1].contiguous()), path)
    with pytest.raises(ValueError, match="ws must be"):
        layer_file.load_layer(path)
    with pytest.raises(ValueError):
        layer_file.save_layer(path, wq, ws.float(), t)


@pytest.mark.gpu
def test_device_pipeline_equals_cpu_pipeline(tmp_path):
    """compute_wush_transform + transform_weights + _C.quant_int4 on the GPU against the CPU pipeline
    with the torch reference quantiser, on the same seeded layer.  The fp64 solve differs between the
    two linear-algebra back ends in the last bits, so T is compared as the bf16 tensor the kernels
    consume, and the codes and scales are compared on the SAME T (the CPU one): there the device
    pipeline must be bit-identical."""
    assert torch.cuda.is_available()
    from my_int4 import _C
    from wush_int4_kernel_b200 import layer_file, wush_transform as wt

    W, x_cal, (wq, ws, t, t64) = _small_layer(seed=9, K=1024, N=320)
    dev = torch.device("cuda:0")
    wq_d, ws_d, t_d, t64_d = layer_file.prepare_layer(W.to(dev), x_cal.to(dev), quantiser=_C.quant_int4, rows_per_block=128)
    rel = ((t64_d.cpu() - t64).norm() / t64.norm()).item()
    assert rel < 1e-6, rel                   # two SVD back ends; the vectors' signs are canonical
    assert (t_d.cpu().view(torch.int16) != t.view(torch.int16)).float().mean().item() < 1e-3   # bf16 roundings of T that flip
    q, s = _C.quant_int4(wt.transform_weights(W.to(dev), t64.to(dev)).to(torch.bfloat16).contiguous())
    w_cpu = wt.transform_weights(W, t64).to(torch.bfloat16)
    same_input = torch.equal(wt.transform_weights(W.to(dev), t64.to(dev)).to(torch.bfloat16).cpu().view(torch.int16),
                             w_cpu.view(torch.int16))
    if same_input:                                                     # identical transformed weights: identical file
        assert torch.equal(q.cpu(), wq) and torch.equal(s.cpu().view(torch.int16), ws.view(torch.int16))
    # in every case: the device quantiser on the CPU pipeline's transformed weights is bit-exact
    q2, s2 = _C.quant_int4(w_cpu.to(dev).contiguous())
    assert torch.equal(q2.cpu(), wq) and torch.equal(s2.cpu().view(torch.int16), ws.view(torch.int16))
    path = str(tmp_path / "gpu_layer.pt")
    layer_file.save_layer(path, wq_d, ws_d, t_d, meta={"device": "cuda"})
    back = layer_file.load_layer(path, device=dev)
    assert back.wq.is_cuda and torch.equal(back.wq, wq_d) and torch.equal(back.ws, ws_d) and torch.equal(back.t_bf16, t_d)
