"""The incrementally written safetensors file is an ordinary safetensors file."""

from concurrent.futures import ThreadPoolExecutor

import pytest
import torch
from safetensors.torch import load_file

from bergson_b200.utils.streamed_safetensors import StreamedSafetensors


def test_threads_write_in_any_order(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {
        "b.weight": torch.randn(7, 13, generator=g),
        "a.weight": torch.randn(5, 3, generator=g).to(torch.bfloat16),
        "c.idx": torch.arange(11, dtype=torch.int64),
        "empty": torch.zeros(0, 4),
        "half": torch.randn(9, generator=g).to(torch.float16),
    }
    path = tmp_path / "x.safetensors"
    with StreamedSafetensors(path, {k: (v.shape, v.dtype) for k, v in tensors.items()}) as w:
        with ThreadPoolExecutor(3) as pool:
            list(pool.map(lambda k: w.write(k, tensors[k].T.contiguous().T if tensors[k].dim() == 2 else tensors[k]),
                          reversed(list(tensors))))
        assert not path.exists()  # published only when complete
    back = load_file(str(path))
    assert set(back) == set(tensors)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and torch.equal(back[k], v), k


def test_missing_or_wrong_tensor_is_an_error(tmp_path):
    path = tmp_path / "y.safetensors"
    w = StreamedSafetensors(path, {"a": ((2, 2), torch.float32), "b": ((3,), torch.float32)})
    w.write("a", torch.ones(2, 2))
    with pytest.raises(ValueError):
        w.write("a", torch.ones(2, 2))
    with pytest.raises(ValueError):
        w.write("b", torch.ones(4))
    with pytest.raises(RuntimeError, match="never written"):
        w.close()
    assert not path.exists() and not (tmp_path / "y.safetensors.partial").exists()
