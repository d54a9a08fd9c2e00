"""Training-time gradient store: the callback's event handlers driven by a minimal
training loop (the HF ``Trainer`` itself needs ``accelerate``, which may be absent)."""

from types import SimpleNamespace

import numpy as np
import torch

from bergson_b200 import load_gradients
from bergson_b200.gradients import AdamNormalizer, GradientProcessor
from bergson_b200.huggingface import GradientCollectorCallback

from .helpers import tiny_dataset, tiny_model


def test_callback_writes_per_example_rows_and_refreshes_normalizers(tmp_path):
    torch.manual_seed(0)
    model = tiny_model("llama")
    model.requires_grad_(True)
    model.train()
    ds = tiny_dataset(n=8, length=10, ragged=False)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    cb = GradientCollectorCallback(tmp_path / "grads", projection_dim=4, dtype=np.dtype(np.float32), track_order=True)
    args = SimpleNamespace(__gradient_collection_enabled__=True)
    state = SimpleNamespace(epoch=0.0, global_step=0)
    loader = SimpleNamespace(dataset=ds)

    cb.on_train_begin(args, state, None, model=model)
    cb.on_epoch_begin(args, state, None, train_dataloader=loader)
    for start in (0, 4):
        idx = torch.arange(start, start + 4)
        x = torch.tensor(ds[idx.tolist()]["input_ids"])
        loss = model(input_ids=x, labels=x, _idx=idx).loss  # the pre-forward hook pops _idx
        loss.backward()
        opt.step()
        opt.zero_grad()
        state.global_step += 1
        cb.on_step_end(args, state, None, model=model, optimizer=opt)
    state.epoch = 1.0
    cb.on_epoch_end(args, state, None)
    cb.on_train_end(args, state, None)

    store = tmp_path / "grads" / "train" / "epoch_0"
    g = np.asarray(load_gradients(store))
    assert g.shape == (8, 14 * 16) and np.isfinite(g).all() and (np.abs(g).sum(1) > 0).all()
    proc = GradientProcessor.load(store)
    assert proc.projection_dim == 4 and len(proc.normalizers) == 14
    assert all(isinstance(n, AdamNormalizer) for n in proc.normalizers.values())
    from datasets import Dataset

    order = Dataset.load_from_disk(str(tmp_path / "grads" / "order.hf"))
    assert sorted(order["_idx"]) == list(range(8)) and set(order["global_step"]) == {1, 2}
    # hooks are gone after training
    assert not any(hasattr(m, "_name") for m in model.modules())


def _drive(cb, model, ds, lr=1e-3, steps=((0, 4), (4, 8))):
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    args = SimpleNamespace(__gradient_collection_enabled__=True)
    state = SimpleNamespace(epoch=0.0, global_step=0)
    cb.on_train_begin(args, state, None, model=model)
    cb.on_epoch_begin(args, state, None, train_dataloader=SimpleNamespace(dataset=ds))
    for lo, hi in steps:
        idx = torch.arange(lo, hi)
        x = torch.tensor(ds[idx.tolist()]["input_ids"])
        model(input_ids=x, labels=x, _idx=idx).loss.backward()
        opt.step()
        opt.zero_grad()
        state.global_step += 1
        cb.on_step_end(args, state, None, model=model, optimizer=opt)
    normalizers = dict(cb.collector.processor.normalizers)
    state.epoch = 1.0
    cb.on_epoch_end(args, state, None)
    cb.on_train_end(args, state, None)
    return normalizers, opt


def test_scale_by_lr_divides_the_second_moments_by_lr_squared(tmp_path):
    """With ``scale_by_lr`` a normalised gradient is ``lr * g / sqrt(v)``, the size of the
    optimizer's own update."""
    ds = tiny_dataset(n=8, length=10, ragged=False)
    got = {}
    for flag in (False, True):
        torch.manual_seed(0)
        model = tiny_model("llama")
        model.requires_grad_(True)
        cb = GradientCollectorCallback(tmp_path / f"g{flag}", projection_dim=4, dtype=np.dtype(np.float32), scale_by_lr=flag)
        got[flag], _ = _drive(cb, model, ds, lr=1e-2)
    assert got[False] and set(got[False]) == set(got[True])
    for name, norm in got[True].items():
        torch.testing.assert_close(norm.weight_avg_sq * 1e-2**2, got[False][name].weight_avg_sq, rtol=1e-5, atol=1e-12)
    g = torch.randn_like(next(iter(got[True].values())).weight_avg_sq)
    a, b = next(iter(got[True].values())), next(iter(got[False].values()))
    torch.testing.assert_close(a.normalize_weight(g.clone(), eps=0.0), 1e-2 * b.normalize_weight(g.clone(), eps=0.0), rtol=1e-4, atol=1e-6)


def test_transposed_layers_get_out_by_in_normalizers_and_no_order_file(tmp_path):
    """GPT-2 style layers store their weight [in, out]; the live normalisers use [out, in], the
    layout of the collected gradients, like the ones read from an optimizer checkpoint."""
    from bergson_b200.models.common import Conv1D

    torch.manual_seed(0)
    model = tiny_model("gpt2")
    model.requires_grad_(True)
    ds = tiny_dataset(n=8, length=10, ragged=False)
    cb = GradientCollectorCallback(tmp_path / "grads", projection_dim=4, dtype=np.dtype(np.float32), track_order=False)
    normalizers, _ = _drive(cb, model, ds)
    base = model.base_model
    checked = 0
    for name, norm in normalizers.items():
        mod = base.get_submodule(name)
        if not isinstance(mod, Conv1D):
            continue
        in_f, out_f = mod.weight.shape
        assert isinstance(norm, AdamNormalizer) and norm.weight_avg_sq.shape == (out_f, in_f), name
        norm.normalize_weight(torch.randn(out_f, in_f))
        checked += in_f != out_f
    assert checked > 0
    assert not (tmp_path / "grads" / "order.hf").exists()
    g = np.asarray(load_gradients(tmp_path / "grads" / "train" / "epoch_0"))
    assert g.shape[0] == 8 and (np.abs(g).sum(1) > 0).all()


def test_callback_splits_attention_heads(tmp_path):
    from bergson_b200.config import AttentionConfig

    torch.manual_seed(0)
    model = tiny_model("llama")
    model.requires_grad_(True)
    ds = tiny_dataset(n=4, length=10, ragged=False)
    name = "layers.0.self_attn.q_proj"
    q = model.base_model.get_submodule(name)
    heads = 4
    cfgs = {name: AttentionConfig(num_heads=heads, head_size=q.out_features // heads, head_dim=2)}
    cb = GradientCollectorCallback(tmp_path / "grads", attention_cfgs=cfgs, projection_dim=4, dtype=np.dtype(np.float32),
                                   use_optimizer_state=False)
    _drive(cb, model, ds, steps=((0, 4),))
    import json

    sizes = json.load(open(tmp_path / "grads" / "train" / "epoch_0" / "info.json"))["grad_sizes"]
    assert all(f"{name}.head_{h}" in sizes for h in range(heads)) and name not in sizes
    g = np.asarray(load_gradients(tmp_path / "grads" / "train" / "epoch_0"))
    assert g.shape == (4, sum(sizes.values())) and np.isfinite(g).all()
