"""Views of a gradient store: rows wider than 2 GiB, module-keyed columns, per-token stores
read through the same calls, and normalisers surviving a save / load."""

import numpy as np
import torch

from bergson_b200.data import create_index, create_token_index, load_gradients, load_module_gradients
from bergson_b200.gradients import AdafactorNormalizer, AdamNormalizer, GradientProcessor


def test_rows_wider_than_two_gib(tmp_path):
    """Unprojected gradients of a billion-parameter model: one row exceeds the 2^31 - 1 bytes that a
    structured record may have, so the store is one flat matrix (a sparse file here)."""
    sizes = {f"layer_{i}.weight": 50_000_000 for i in range(12)}
    assert sum(sizes.values()) * 4 > 2**31
    create_index(tmp_path, num_grads=3, grad_sizes=sizes, dtype=np.float32)
    mm = load_gradients(tmp_path)
    assert mm.shape == (3, sum(sizes.values()))
    by_module = load_module_gradients(tmp_path)
    assert len(by_module) == 3 and list(by_module.keys()) == list(sizes)
    assert by_module["layer_3.weight"].shape == (3, 50_000_000)


def test_module_columns_of_document_and_token_stores(tmp_path):
    sizes = {"a.weight": 3, "b.weight": 5}
    rng = np.random.default_rng(0)
    buf = create_index(tmp_path / "doc", num_grads=4, grad_sizes=sizes, dtype=np.float32)
    want = rng.standard_normal((4, 8)).astype(np.float32)
    buf[:] = want
    buf.flush()
    g = load_module_gradients(tmp_path / "doc")
    np.testing.assert_array_equal(g["a.weight"], want[:, :3])
    np.testing.assert_array_equal(g["b.weight"], want[:, 3:])
    tok, offsets = create_token_index(tmp_path / "tok", np.array([2, 3, 1]), sizes, np.float32)
    rows = rng.standard_normal((int(offsets[-1]), 8)).astype(np.float32)
    tok[:] = rows
    tok.flush()
    assert load_gradients(tmp_path / "tok").shape == (6, 8)
    np.testing.assert_array_equal(np.asarray(load_gradients(tmp_path / "tok")), rows)
    gt = load_module_gradients(tmp_path / "tok")
    assert len(gt) == 6
    np.testing.assert_array_equal(gt["a.weight"], rows[:, :3])


def test_normalisers_survive_save_and_load(tmp_path):
    w, b = torch.rand(4, 8), torch.rand(4)
    GradientProcessor(normalizers={"layer": AdamNormalizer(weight_avg_sq=w, bias_avg_sq=b)}, include_bias=True).save(tmp_path / "adam")
    got = GradientProcessor.load(tmp_path / "adam").normalizers["layer"]
    assert isinstance(got, AdamNormalizer)
    torch.testing.assert_close(got.weight_avg_sq, w)
    torch.testing.assert_close(got.bias_avg_sq, b)
    ada = AdafactorNormalizer(row=torch.rand(4), col=torch.rand(8), bias_avg_sq=b)
    GradientProcessor(normalizers={"layer": ada}, include_bias=True).save(tmp_path / "ada")
    back = GradientProcessor.load(tmp_path / "ada")
    got = back.normalizers["layer"]
    assert isinstance(got, AdafactorNormalizer) and back.include_bias
    torch.testing.assert_close(got.row, ada.row)
    torch.testing.assert_close(got.col, ada.col)
    torch.testing.assert_close(got.bias_avg_sq, b)
    none = AdafactorNormalizer(row=torch.rand(4), col=torch.rand(8))
    GradientProcessor(normalizers={"layer": none}).save(tmp_path / "nobias")
    assert GradientProcessor.load(tmp_path / "nobias").normalizers["layer"].bias_avg_sq is None
