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
