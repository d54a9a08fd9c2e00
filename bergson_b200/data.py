"""Datasets, batching and the on-disk gradient / score stores.

On-disk layouts (byte-compatible with the reference, ``bergson/data.py``):

* gradient store: ``gradients.bin`` = C-order ``(num_grads, sum(grad_sizes))`` array of
  ``base_dtype`` + ``info.json``; per-token stores add ``offsets.npy``;
* score store: ``scores.bin`` = structured records of ``(score_i, written_i)`` pairs +
  ``info.json`` (see ``score/score_writer.py``).
"""

from __future__ import annotations

import heapq
import json
import math
import os
import random
import re
from pathlib import Path
from typing import Any, Iterator, Sequence
from urllib.parse import parse_qsl

import ml_dtypes  # noqa: F401  (registers bfloat16 with numpy)
import numpy as np
import torch
import torch.distributed as dist
from datasets import Dataset, DatasetDict, concatenate_datasets, load_dataset, load_from_disk
from numpy.lib.recfunctions import structured_to_unstructured

from .config.config import DataConfig, ScoreConfig
from .config.config_io import CONFIG_FILENAME, load_subconfig, read_config
from .utils.utils import assert_type, simple_parse_kwargs_string


def _rank_world() -> tuple[int, int]:
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _data_rank_world() -> tuple[int, int]:
    """(rank, world) for splitting data: the ranks of one tensor-parallel group share data."""
    from .parallel import topology

    return topology.data_rank_world()


# --------------------------------------------------------------------------- #
# synthetic data
# --------------------------------------------------------------------------- #


def zipf_token_ids(
    n: int, length: int, vocab: int, seed: int = 0, s: float = 1.1, min_length: int | None = None
) -> list[list[int]]:
    """``n`` sequences of token ids with ``P(id = k) ~ (k+1)^-s`` over ``[0, vocab)``.

    Drawn by inverse-CDF lookup from a seeded ``numpy`` PCG64 stream, so the data is
    identical on every machine.  ``min_length`` < ``length`` gives ragged lengths
    (uniform in ``[min_length, length]``).
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    cdf = np.cumsum(1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s))
    cdf /= cdf[-1]
    if min_length is None or min_length >= length:
        lens = np.full(n, length, dtype=np.int64)
    else:
        lens = rng.integers(min_length, length + 1, size=n)
    flat = np.searchsorted(cdf, rng.random(int(lens.sum())), side="left").astype(np.int64)
    np.minimum(flat, vocab - 1, out=flat)
    out, pos = [], 0
    for L in lens:
        out.append(flat[pos : pos + L].tolist())
        pos += int(L)
    return out


def synthetic_dataset(spec: str) -> Dataset:
    """``synthetic:zipf?n=2048&len=256&vocab=50304&seed=0[&min_len=..][&s=1.1]``."""
    body = spec[len("synthetic:"):]
    kind, _, query = body.partition("?")
    if kind != "zipf":
        raise ValueError(f"Unknown synthetic dataset kind {kind!r}")
    o = dict(parse_qsl(query))
    ids = zipf_token_ids(
        int(o.get("n", 1024)),
        int(o.get("len", 256)),
        int(o.get("vocab", 50304)),
        int(o.get("seed", 0)),
        float(o.get("s", 1.1)),
        int(o["min_len"]) if "min_len" in o else None,
    )
    return Dataset.from_dict({"input_ids": ids, "length": [len(x) for x in ids]})


def _slice_rows(ds: Dataset, split: str) -> Dataset:
    """Apply a ``name[a:b]`` row slice (absolute indices or percentages) to ``ds``."""
    m = re.fullmatch(r"[^\[]*\[\s*(-?\d+%?)?\s*:\s*(-?\d+%?)?\s*\]", split.strip())
    if not m:
        return ds
    n = len(ds)

    def pos(tok, default):
        if tok is None:
            return default
        v = int(tok.rstrip("%"))
        v = v * n // 100 if tok.endswith("%") else v
        return max(0, min(n, v + n if v < 0 else v))

    return ds.select(range(pos(m.group(1), 0), pos(m.group(2), n)))


def load_data_string(data_str: str, split: str = "train", subset: str | None = None, data_kwargs: str = "") -> Dataset:
    """Resolve a dataset string to a ``datasets.Dataset``."""
    if data_str.startswith("synthetic:"):
        return _slice_rows(synthetic_dataset(data_str), split)
    p = Path(data_str)
    if data_str.endswith(".csv"):
        ds = load_dataset("csv", data_files=data_str, split=split)
    elif data_str.endswith((".json", ".jsonl")):
        ds = load_dataset("json", data_files=data_str, split=split)
    elif p.is_dir() and ((p / "dataset_info.json").exists() or (p / "dataset_dict.json").exists() or (p / "state.json").exists()):
        ds = load_from_disk(data_str, keep_in_memory=False)
        if isinstance(ds, DatasetDict):
            ds = ds[split.split("[")[0]]
        return _slice_rows(assert_type(Dataset, ds), split)
    else:
        try:
            ds = load_dataset(data_str, subset, split=split, **simple_parse_kwargs_string(data_kwargs))
        except ValueError as e:
            if "load_from_disk" not in str(e):
                raise
            ds = load_from_disk(data_str, keep_in_memory=False)
    if isinstance(ds, DatasetDict):
        if "[" in split or "+" in split:
            raise NotImplementedError(
                f"Split slicing/concatenation expressions are not supported for load_from_disk paths: {split!r}"
            )
        ds = ds[split]
    return assert_type(Dataset, ds)


# --------------------------------------------------------------------------- #
# token bookkeeping
# --------------------------------------------------------------------------- #


def compute_num_token_grads(data: Dataset) -> np.ndarray:
    """Per-example count of per-token gradient rows: ``max(length - 1, 0)`` — every
    non-padding position except the last, regardless of label masking."""
    cols = data.column_names
    if "length" in cols:
        lengths = np.asarray(data["length"], dtype=np.int64)
    else:
        col = "input_ids" if "input_ids" in cols else "labels"
        lengths = np.asarray([len(x) for x in data[col]], dtype=np.int64)
    return np.maximum(lengths - 1, 0)


def ceildiv(a: int, b: int) -> int:
    return -(-a // b)


# --------------------------------------------------------------------------- #
# batching
# --------------------------------------------------------------------------- #


def _allocate_batches_world(
    doc_lengths: Sequence[int],
    N: int,
    world_size: int,
    seed: int = 42,
    ranks: list[int] | None = None,
    max_batch_size: int | None = None,
) -> list[list[list[int]]]:
    """Greedy length-sorted packing under ``max_len * n_docs <= N`` for every rank.

    Documents shorter than two tokens are left out (their store rows stay zero).
    Batches are split until their count is a positive multiple of ``world_size``,
    dealt round-robin, and each requested rank's list is shuffled with ``seed``.
    """
    ranks = list(range(world_size)) if ranks is None else ranks
    order = sorted(
        (i for i, l in enumerate(doc_lengths) if l >= 2), key=lambda i: doc_lengths[i], reverse=True
    )
    skipped = len(doc_lengths) - len(order)
    if skipped and _rank_world()[0] == 0:
        print(f"Skipping {skipped} documents with fewer than 2 tokens (no valid next-token labels).")
    if len(order) < world_size:
        raise RuntimeError("Not enough documents (with 2+ tokens) to distribute across workers.")
    if doc_lengths[order[0]] > N:
        raise RuntimeError(f"At least one document is too long for the token batch size {N}.")

    batches: list[list[int]] = []
    cur: list[int] = []
    for i in order:
        if cur:
            head = doc_lengths[cur[0]]  # longest in the batch (sorted descending)
            fits = max(head, doc_lengths[i]) * (len(cur) + 1) <= N
            if fits and (max_batch_size is None or len(cur) < max_batch_size):
                cur.append(i)
                continue
            batches.append(cur)
        cur = [i]
    if cur:
        batches.append(cur)

    if len(batches) < world_size:
        # Peel singletons off the largest batches until every rank has one.
        heap = [(-len(b), n, b) for n, b in enumerate(batches)]
        heapq.heapify(heap)
        tick = len(heap)
        while len(heap) < world_size:
            _, _, big = heapq.heappop(heap)
            if len(big) == 1:
                raise RuntimeError("Not enough documents to give each worker at least one batch.")
            single = [big.pop()]
            heapq.heappush(heap, (-len(big), tick, big))
            heapq.heappush(heap, (-1, tick + 1, single))
            tick += 2
        batches = [b for _, _, b in heap]

    target = world_size * ceildiv(len(batches), world_size)
    i = 0
    while len(batches) < target and i < len(batches):
        b = batches[i % len(batches)]
        if len(b) > 1:
            batches.append([b.pop()])
        i += 1
    assert len(batches) == target, (
        "Could not construct a number of batches divisible by the world size. If variability of "
        "item lengths in your dataset is low consider using a different dataset size or token batch size."
    )
    assert all(max(doc_lengths[i] for i in b) * len(b) <= N for b in batches)

    alloc: list[list[list[int]]] = [batches[r::world_size] for r in range(world_size)]
    assert len({len(a) for a in alloc}) == 1
    for r in ranks:
        random.seed(seed)
        random.shuffle(alloc[r])
    return [alloc[r] for r in ranks]


def allocate_batches(
    doc_lengths: Sequence[int], N: int, seed: int = 42, max_batch_size: int | None = None
) -> list[list[int]]:
    """This rank's batches (see ``_allocate_batches_world``)."""
    rank, world = _data_rank_world()
    (mine,) = _allocate_batches_world(doc_lengths, N, world, seed, ranks=[rank], max_batch_size=max_batch_size)
    return mine


def pad_and_tensor(
    sequences: list[list[int]],
    labels: list[list[int]] | None = None,
    *,
    padding_value: int = 0,
    dtype: torch.dtype | None = torch.long,
    device: torch.device | None = None,
    sync_max_len: bool = True,
    pinned: bool = False,
):
    """Right-pad to a common length and return ``(tokens, labels, shift_loss_mask,
    collection_mask)``.  Label padding is -100.  ``shift_loss_mask[i, t]`` says that
    position ``t`` predicts a supervised token; ``collection_mask`` marks every real
    position except each sequence's last.  With ``sync_max_len`` the pad length is the
    maximum over ranks (needed when activations must have equal shapes everywhere).
    ``pinned`` (B200) stages the host tensors in page-locked memory so the copy to
    ``device`` is asynchronous.
    """
    labels = sequences if labels is None else labels
    lens = [len(s) for s in sequences]
    S = max(lens)
    if sync_max_len and dist.is_initialized():
        t = torch.tensor(S, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        S = int(t)
    n = len(sequences)
    tok = np.full((n, S), padding_value, dtype=np.int64)
    lab = np.full((n, S), -100, dtype=np.int64)
    for r, (s, l) in enumerate(zip(sequences, labels)):
        tok[r, : len(s)] = s
        lab[r, : len(l)] = l
    tok_t, lab_t = torch.from_numpy(tok), torch.from_numpy(lab)
    if dtype is not None and dtype != torch.long:
        tok_t, lab_t = tok_t.to(dtype), lab_t.to(dtype)
    lens_t = torch.tensor(lens)
    if device is not None and torch.device(device).type == "cuda":
        if pinned:
            tok_t, lab_t, lens_t = tok_t.pin_memory(), lab_t.pin_memory(), lens_t.pin_memory()
        tok_t = tok_t.to(device, non_blocking=pinned)
        lab_t = lab_t.to(device, non_blocking=pinned)
        lens_t = lens_t.to(device, non_blocking=pinned)
    shift = torch.zeros(n, S, dtype=torch.bool, device=tok_t.device)
    shift[:, :-1] = lab_t[:, 1:] != -100
    pos = torch.arange(S, device=tok_t.device)
    collect = (pos[None, :] + 1) < lens_t[:, None]
    return tok_t, lab_t, shift, collect


# --------------------------------------------------------------------------- #
# gradient store
# --------------------------------------------------------------------------- #


def column_offsets(grad_sizes: dict[str, int]) -> dict[str, tuple[int, int]]:
    """Module name -> ``(start, end)`` column range, modules in ``grad_sizes`` order."""
    out, start = {}, 0
    for name, size in grad_sizes.items():
        out[name] = (start, start + size)
        start += size
    return out


def _allocate_file(path: Path, nbytes: int) -> None:
    with open(path, "wb") as f:
        f.truncate(nbytes)
        os.fsync(f.fileno())


def create_index(root: Path, num_grads: int, grad_sizes: dict[str, int], dtype) -> np.memmap:
    """Create (rank 0) and map (all ranks) a ``(num_grads, total_dim)`` store."""
    root = Path(root)
    np_dtype = np.dtype(dtype)
    width = sum(grad_sizes.values())
    rank, _ = _rank_world()
    if rank == 0:
        root.mkdir(parents=True, exist_ok=True)
        _allocate_file(root / "gradients.bin", np_dtype.itemsize * width * num_grads)
        with (root / "info.json").open("w") as f:
            json.dump(
                {
                    "attribute_tokens": False,
                    "num_items": num_grads,
                    "num_grads": num_grads,
                    "grad_sizes": grad_sizes,
                    "base_dtype": np_dtype.name,
                },
                f,
                indent=2,
            )
    if dist.is_initialized():
        dist.barrier()
    return np.memmap(root / "gradients.bin", dtype=np_dtype, mode="r+", shape=(num_grads, width))


def create_token_index(root: Path, num_token_grads: np.ndarray, grad_sizes: dict[str, int], dtype):
    """Ragged per-token store: rows ``offsets[i]:offsets[i+1]`` belong to example i."""
    root = Path(root)
    np_dtype = np.dtype(dtype)
    width = sum(grad_sizes.values())
    offsets = np.zeros(len(num_token_grads) + 1, dtype=np.int64)
    np.cumsum(num_token_grads, out=offsets[1:])
    total = int(offsets[-1])
    rank, _ = _rank_world()
    if rank == 0:
        root.mkdir(parents=True, exist_ok=True)
        _allocate_file(root / "gradients.bin", np_dtype.itemsize * width * total)
        np.save(root / "offsets.npy", offsets)
        with (root / "info.json").open("w") as f:
            json.dump(
                {
                    "attribute_tokens": True,
                    "num_items": len(num_token_grads),
                    "num_grads": total,
                    "grad_sizes": grad_sizes,
                    "base_dtype": np_dtype.name,
                },
                f,
                indent=2,
            )
    if dist.is_initialized():
        dist.barrier()
    mm = np.memmap(root / "gradients.bin", dtype=np_dtype, mode="r+", shape=(total, width))
    return mm, offsets


def load_gradients(root_dir: Path | str) -> np.memmap:
    """Read-only map of a store as ``(num_grads, total_dim)``."""
    root_dir = Path(root_dir)
    with (root_dir / "info.json").open() as f:
        info = json.load(f)
    if "base_dtype" in info:
        dtype = np.dtype(info["base_dtype"])
    else:  # stores written before ``base_dtype`` existed
        dtype = np.dtype(info["dtype"]["formats"][0]).base
    return np.memmap(
        root_dir / "gradients.bin",
        dtype=dtype,
        mode="r",
        shape=(info["num_grads"], sum(info["grad_sizes"].values())),
    )


def load_token_gradients(root_dir: Path | str):
    root_dir = Path(root_dir)
    mm = load_gradients(root_dir)
    offsets = np.load(root_dir / "offsets.npy")
    return mm, np.diff(offsets).astype(np.int64), offsets


class TokenGradients:
    """``tg[i]`` -> ``(num_token_grads[i], total_dim)`` rows of example i."""

    def __init__(self, root_dir: Path | str):
        self.mmap, self._counts, self._offsets = load_token_gradients(root_dir)

    @property
    def num_token_grads(self) -> np.ndarray:
        return self._counts

    def __len__(self) -> int:
        return len(self._counts)

    def __getitem__(self, i: int) -> np.ndarray:
        return np.asarray(self.mmap[self._offsets[i] : self._offsets[i + 1]])


class ModuleGradients:
    """Mapping-like per-module column views over a flat store."""

    def __init__(self, mmap: np.memmap, grad_sizes: dict[str, int]):
        self.mmap = mmap
        self.offsets = column_offsets(grad_sizes)

    def __getitem__(self, name: str) -> np.ndarray:
        lo, hi = self.offsets[name]
        return self.mmap[:, lo:hi]

    def __len__(self) -> int:
        return len(self.mmap)

    def __iter__(self) -> Iterator[str]:
        return iter(self.offsets)

    def __contains__(self, name: str) -> bool:
        return name in self.offsets

    def keys(self):
        return self.offsets.keys()


def load_module_gradients(root_dir: Path | str) -> ModuleGradients:
    root_dir = Path(root_dir)
    with (root_dir / "info.json").open() as f:
        sizes = json.load(f)["grad_sizes"]
    return ModuleGradients(load_gradients(root_dir), sizes)


def load_gradient_dataset(root_dir: Path) -> Dataset:
    """``data.hf`` joined with a ``gradients`` fixed-size-list column (bf16 -> fp32)."""
    import pyarrow as pa

    def one(d: Path) -> Dataset:
        ds = Dataset.load_from_disk(str(d / "data.hf"))
        mm = load_gradients(d)
        flat = mm.reshape(-1).copy()
        if flat.dtype == np.dtype("bfloat16"):
            flat = flat.astype(np.float32)
        col = pa.FixedSizeListArray.from_arrays(pa.array(flat), mm.shape[1])
        return ds.add_column("gradients", col, new_fingerprint="gradients")

    root_dir = Path(root_dir)
    if (root_dir / "data.hf").exists():
        return one(root_dir)
    parts = [one(p) for p in sorted(root_dir.iterdir()) if p.is_dir()]
    return concatenate_datasets(parts).flatten_indices()


# --------------------------------------------------------------------------- #
# score store (reader side)
# --------------------------------------------------------------------------- #


class Scores:
    """Reader of ``scores.bin``.  ``offsets`` is set for per-token stores."""

    def __init__(self, mmap: np.memmap, info: dict[str, Any], offsets=None):
        self.mmap, self.info, self.offsets = mmap, info, offsets
        self.num_scores = info["num_scores"]
        self._fields = [f"score_{i}" for i in range(self.num_scores)]

    def __len__(self) -> int:
        return self.info["num_items"]

    def __getitem__(self, key):
        return structured_to_unstructured(self.mmap[key][self._fields])

    def get(self, key, score_idx: int = 0):
        return self.mmap[key][f"score_{score_idx}"]

    def is_written(self) -> bool:
        return all(bool(np.all(self.mmap[f"written_{i}"])) for i in range(self.num_scores))

    def to_grid(self) -> torch.Tensor:
        """Per-token store -> zero-padded ``[docs, seq_len(, num_scores)]``."""
        assert self.offsets is not None, "to_grid() requires a per-token store"
        counts = np.diff(self.offsets).astype(np.int64)
        grid = np.zeros((len(self), int(counts.max()) + 1, self.num_scores), dtype=np.float32)
        for d in range(len(self)):
            grid[d, : counts[d]] = self[self.offsets[d] : self.offsets[d + 1]]
        t = torch.from_numpy(grid)
        return t[..., 0] if self.num_scores == 1 else t


def load_scores(path: Path) -> Scores:
    path = Path(path)
    with open(path / "info.json") as f:
        info = json.load(f)
    mm = np.memmap(path / "scores.bin", dtype=info["dtype"], mode="r", shape=(info["num_rows"],))
    offsets = np.load(path / "offsets.npy") if info.get("attribute_tokens") else None
    return Scores(mm, info, offsets)


def _load_legacy_pt_scores(score_path: str):
    scores = torch.load(score_path, map_location="cpu")
    if not isinstance(scores, torch.Tensor) or scores.ndim not in (2, 3):
        return scores, False
    if scores.ndim == 3:
        return scores, True
    cfg_path = Path(score_path).parent / CONFIG_FILENAME
    if not cfg_path.is_file():
        return scores, False
    try:
        steps = read_config(cfg_path)["steps"]
    except Exception:
        return scores, False
    for step in steps:
        for body in step.values():
            if isinstance(body, dict):
                return scores, body.get("query_method") == "none"
    return scores, False


def load_scores_loss_signed(score_path: str):
    """Scores in the convention "negative = lowers the query loss".  Stores whose
    sibling ``config.yaml`` says ``higher_is_better`` are negated.  Returns
    ``(scores, is_multi_query)``."""
    if str(score_path).endswith(".pt"):
        return _load_legacy_pt_scores(str(score_path))
    loaded = load_scores(Path(score_path))
    cfg = load_subconfig(score_path, "score_cfg", ScoreConfig)
    if loaded.offsets is not None:
        scores = loaded.to_grid()
    else:
        arr = np.asarray(loaded[:])
        dt = arr.dtype if np.issubdtype(arr.dtype, np.floating) else np.float32
        scores = torch.from_numpy(arr.astype(dt, copy=True))
    if cfg is not None and cfg.higher_is_better:
        scores = -scores
    return scores, loaded.num_scores > 1


def sorted_checkpoints(folder: str) -> list[tuple[int, str]]:
    """``[(step, path)]`` of ``step_<i>.ckpt`` entries, ascending."""
    pat = re.compile(r"step_(\d+)\.ckpt$")
    found = []
    for name in os.listdir(folder):
        if m := pat.match(name):
            found.append((int(m.group(1)), os.path.join(folder, name)))
    return sorted(found)


# --------------------------------------------------------------------------- #
# tokenisation
# --------------------------------------------------------------------------- #


def tokenize(batch: dict, *, args: DataConfig, tokenizer, max_length: int | None = None):
    """Tokenise a batch.  Plain text: ids only.  Prompt/completion or conversation
    data: rendered through the chat template with labels -100 outside assistant
    spans (spans located right-to-left by ``rfind`` so repeated text resolves to the
    last occurrence)."""
    kw: dict[str, Any] = dict(return_attention_mask=False, return_length=True, truncation=args.truncation)
    if args.truncation and max_length is not None:
        kw["max_length"] = max_length
    if args.completion_column:
        convos = [
            [
                {"role": "user", "content": assert_type(str, p)},
                {"role": "assistant", "content": assert_type(str, c)},
            ]
            for p, c in zip(batch[args.prompt_column], batch[args.completion_column])
        ]
    elif args.conversation_column:
        convos = assert_type(list, batch[args.conversation_column])
    else:
        return tokenizer(batch[args.prompt_column], **kw)

    texts = tokenizer.apply_chat_template(convos, tokenize=False)
    enc = tokenizer(texts, add_special_tokens=False, **kw)
    all_labels = []
    for i, convo in enumerate(convos):
        text, limit, spans = texts[i], len(texts[i]), []
        for msg in reversed(convo):
            if msg["role"] != "assistant":
                continue
            ans = msg["content"]
            start = text.rfind(ans, 0, limit)
            if start < 0:
                raise RuntimeError(
                    "Failed to find completion in the chat-formatted conversation. Make sure the "
                    "chat template does not alter the completion, e.g. by removing leading whitespace."
                )
            end = start + len(ans)
            s_tok = enc.char_to_token(i, start)
            e_tok = enc.char_to_token(i, end)
            if e_tok is None and end > 0:
                prev = enc.char_to_token(i, end - 1)
                e_tok = prev + 1 if prev is not None else None
            spans.append((s_tok, e_tok))
            limit = start
        ids = enc["input_ids"][i]
        lab = [-100] * len(ids)
        for s_tok, e_tok in reversed(spans):
            if s_tok is None:  # span lies beyond the truncation point
                continue
            e_tok = len(ids) if e_tok is None else e_tok
            lab[s_tok:e_tok] = ids[s_tok:e_tok]
        all_labels.append(lab)
    return dict(**enc, labels=all_labels)


def tokenize_and_chunk(dataset: Dataset, tokenizer, chunk_size: int, text_column: str = "text", *, num_proc: int | None = None) -> Dataset:
    """EOS-joined token stream cut into ``chunk_size`` windows, with a parallel
    ``doc_ids`` column mapping every token to its source row."""
    eos = tokenizer.eos_token_id
    if eos is None:
        raise ValueError("Tokenizer does not have an eos_token_id set.")
    n_before = len(dataset)
    dataset = dataset.map(lambda _, idx: {"_orig_idx": idx}, with_indices=True)
    dataset = dataset.filter(lambda r: isinstance(r[text_column], str) and r[text_column].strip() != "")
    if (dropped := n_before - len(dataset)) > 0:
        print(f"Warning: {dropped}/{n_before} empty documents ({dropped / n_before * 100:.1f}%).")
    if num_proc is None:
        num_proc = min((os.cpu_count() or 2) // 2, max(1, len(dataset) // 256))
    num_proc = max(1, num_proc)

    def tok(batch):
        out = tokenizer(batch[text_column], add_special_tokens=False, truncation=False, padding=False)
        return {"input_ids": out["input_ids"], "_orig_idx": batch["_orig_idx"]}

    tokd = dataset.map(tok, batched=True, num_proc=num_proc if num_proc > 1 else None,
                       remove_columns=[c for c in dataset.column_names if c != "_orig_idx"])

    def chunk(batch):
        toks: list[int] = []
        docs: list[int] = []
        for d, ids in zip(batch["_orig_idx"], batch["input_ids"]):
            toks.extend(ids)
            toks.append(eos)
            docs.extend([d] * (len(ids) + 1))
        k = len(toks) // chunk_size
        return {
            "input_ids": [toks[j * chunk_size : (j + 1) * chunk_size] for j in range(k)],
            "doc_ids": [docs[j * chunk_size : (j + 1) * chunk_size] for j in range(k)],
            "length": [chunk_size] * k,
        }

    num_proc = min(num_proc, max(len(tokd) // (chunk_size * 4), 1))
    bs = max(1, min(10_000, len(tokd) // num_proc))
    return tokd.map(chunk, batched=True, batch_size=bs, num_proc=num_proc if num_proc > 1 else None,
                    remove_columns=tokd.column_names)


def unflatten(x: torch.Tensor, shapes: dict[str, Sequence[int]], dim: int = -1):
    """Split ``x`` along ``dim`` into named tensors of the given shapes."""
    sizes = [math.prod(s) for s in shapes.values()]
    return {n: part.unflatten(dim, s) for (n, s), part in zip(shapes.items(), x.split(sizes, dim=dim))}
