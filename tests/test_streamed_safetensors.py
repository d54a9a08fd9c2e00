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


def test_save_tensors_matches_save_file(tmp_path):
    from bergson_b200.utils.streamed_safetensors import save_tensors

    g = torch.Generator().manual_seed(1)
    tensors = {f"t{i}": torch.randn(17 + i, 9, generator=g) for i in range(7)}
    tensors["wide"] = torch.randn(3, 5, generator=g).to(torch.bfloat16)
    for threads in (1, 4):
        save_tensors(tensors, str(tmp_path / f"x{threads}.safetensors"), threads=threads)
        back = load_file(str(tmp_path / f"x{threads}.safetensors"))
        assert all(torch.equal(back[k], v) for k, v in tensors.items()) and set(back) == set(tensors)


@pytest.mark.gpu
def test_device_tensors_go_through_pinned_staging(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from bergson_b200.utils import streamed_safetensors as ss

    g = torch.Generator("cuda").manual_seed(2)
    # larger than one staging chunk, odd sizes, a strided view, several dtypes
    tensors = {"big": torch.randn(3000, 3001, device="cuda", generator=g),
               "bf": torch.randn(1025, 513, device="cuda", generator=g).to(torch.bfloat16),
               "view": torch.randn(64, 200, device="cuda", generator=g)[:, ::2].contiguous(),
               "idx": torch.arange(1000, device="cuda"), "host": torch.randn(5, 5)}
    assert tensors["big"].numel() * 4 > 2 * ss._CHUNK
    for threads in (1, 3):
        ss.save_tensors(tensors, str(tmp_path / f"d{threads}.safetensors"), threads=threads)
        back = load_file(str(tmp_path / f"d{threads}.safetensors"))
        for k, v in tensors.items():
            assert torch.equal(back[k], v.cpu()), k
    assert 0 < ss._n_slots <= ss._MAX_SLOTS and ss._free_slots.qsize() == ss._n_slots  # every slot was returned


def test_an_exception_leaves_no_file_behind(tmp_path):
    path = tmp_path / "z.safetensors"
    with pytest.raises(KeyError):
        with StreamedSafetensors(path, {"a": ((2,), torch.float32)}) as w:
            w.write("a", torch.ones(2))
            raise KeyError("the producer failed")
    assert not path.exists() and not (tmp_path / "z.safetensors.partial").exists()
    # an older complete file is only replaced by a complete new one
    with StreamedSafetensors(path, {"a": ((2,), torch.float32)}) as w:
        w.write("a", torch.ones(2))
    with pytest.raises(RuntimeError):
        with StreamedSafetensors(path, {"a": ((2,), torch.float32), "b": ((1,), torch.float32)}) as w:
            w.write("a", torch.zeros(2))
    assert torch.equal(load_file(str(path))["a"], torch.ones(2))
