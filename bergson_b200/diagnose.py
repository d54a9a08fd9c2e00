"""``test_model_configuration``: does a document's gradient depend on what it is batched
with?  (reference ``bergson/diagnose.py:311-505``)

Three checks: (1) the chat-template tokenisation of ``data.tokenize`` agrees with
``apply_chat_template(tokenize=True)`` (no duplicated / missing BOS / EOS); (2) a document
batched with random tokens of equal length (no padding) gives the same gradient as alone;
(3) an escalating series of numeric configurations (base precision -> fp32 with TF32 ->
math attention -> fp32 + math attention -> plain fp32) is tried until a document padded
next to a longer one gives the same gradient (cosine above ``threshold``) in every trial.
"""

from __future__ import annotations

import random

import torch
import torch.nn.functional as F

from .config import DataConfig
from .data import load_data_string, pad_and_tensor, tokenize
from .diagnose_config import DiagnoseConfig
from .models import load_model
from .utils.utils import simple_parse_kwargs_string

DTYPE_MAP = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _example_loss(model, x, y, idx: int = 0):
    logits = model(x).logits[:, :-1]
    tgt = y[:, 1:]
    tok = F.cross_entropy(logits.reshape(-1, logits.size(-1)), tgt.flatten(), reduction="none").reshape_as(tgt)
    return tok[idx][tgt[idx] != -100].sum()


def _measure(model, short_ids, long_ids, device) -> tuple[float, float]:
    """(cosine between the gradient of ``short_ids`` alone and batched with ``long_ids``,
    absolute loss difference)."""
    xa, ya, _, _ = pad_and_tensor([short_ids], device=device, sync_max_len=False)
    xm, ym, _, _ = pad_and_tensor([short_ids, long_ids], device=device, sync_max_len=False)
    model.zero_grad()
    la = _example_loss(model, xa, ya)
    la.backward()
    alone = {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    lm = _example_loss(model, xm, ym)
    lm.backward()
    dot = na = nb = 0.0
    for n, p in model.named_parameters():
        if p.grad is not None and n in alone:
            a, b = alone[n].double(), p.grad.detach().double()
            dot += float((a * b).sum())
            na += float((a * a).sum())
            nb += float((b * b).sum())
    return dot / (na**0.5 * nb**0.5 + 1e-12), float((lm.detach() - la.detach()).abs())


def _trials(model, docs, n_trials: int, seed: int, device, vocab: int | None = None):
    """Different-length pairs, or (``vocab`` given) a document next to random tokens of its
    own length."""
    rng = random.Random(seed)
    rows = []
    for t in range(n_trials):
        if vocab is None:
            i, j = rng.sample(range(len(docs)), 2)
            a, b = sorted((docs[i], docs[j]), key=len)
        else:
            a = docs[rng.randrange(len(docs))]
            b = [rng.randrange(vocab) for _ in a]
        cos, dl = _measure(model, a, b, device)
        rows.append({"trial": t, "short_len": len(a), "long_len": len(b), "ratio": len(b) / len(a), "cos_sim": cos,
                     "loss_diff": dl})
    return rows


def _summarise(rows, threshold: float) -> tuple[float, int]:
    cs = torch.tensor([r["cos_sim"] for r in rows])
    flagged = int((cs < threshold).sum())
    print(f"{'trial':>6s} {'short':>6s} {'long':>6s} {'ratio':>6s} {'cos_sim':>10s} {'loss_diff':>12s}")
    for r in rows:
        mark = " <<<" if r["cos_sim"] < threshold else ""
        print(f"{r['trial']:>6d} {r['short_len']:>6d} {r['long_len']:>6d} {r['ratio']:>6.1f} {r['cos_sim']:>10.6f} "
              f"{r['loss_diff']:>12.6f}{mark}")
    print(f"\n  Cos sim:  mean={cs.mean():.6f}  min={cs.min():.6f}  max={cs.max():.6f}")
    print(f"  Flagged:  {flagged}/{len(rows)} trials below {threshold}")
    return float(cs.min()), flagged


def diagnose_special_tokens(model_name: str) -> bool:
    """True when ``tokenize`` reproduces ``apply_chat_template(tokenize=True)`` on a sample
    conversation (or when the model has no chat template / tokenizer)."""
    if model_name.startswith("native:"):
        print("  native model spec: no tokenizer, special token check not applicable.")
        return True
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(model_name)
    msgs = [{"role": "user", "content": "Hello"}, {"role": "assistant", "content": "Hi there"}]
    try:
        truth = list(tok.apply_chat_template(msgs, tokenize=True, add_generation_prompt=False, return_dict=True)["input_ids"])
    except Exception:
        print("  No chat template found - special token check not applicable.")
        return True
    try:
        got = list(tokenize({"conversation": [msgs]}, args=DataConfig(conversation_column="conversation"), tokenizer=tok)["input_ids"][0])
    except Exception as e:  # noqa: BLE001
        print(f"  FAIL: tokenize() raised {type(e).__name__}: {e}")
        return False
    if got == truth:
        print("  PASS: tokenize() matches apply_chat_template(tokenize=True).")
        return True
    print(f"  FAIL: tokenize() gives {len(got)} tokens, expected {len(truth)}")
    for name, tid in (("BOS", tok.bos_token_id), ("EOS", tok.eos_token_id)):
        if tid is not None and got.count(tid) != truth.count(tid):
            kind = "DUPLICATED" if got.count(tid) > truth.count(tid) else "MISSING"
            print(f"    <<< {kind} {name} (id={tid}): got {got.count(tid)}, expected {truth.count(tid)}")
    return False


def _load_docs(cfg: DiagnoseConfig) -> tuple[list[list[int]], int]:
    ds = load_data_string(cfg.dataset, cfg.split)
    if "input_ids" in ds.column_names:
        rows = ds["input_ids"]
        vocab = max(max(r) for r in rows) + 1
    else:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(cfg.model)
        rows = [tok(t)["input_ids"] for t in ds["text"]]
        vocab = tok.vocab_size
    docs = [r[: cfg.max_len] for r in rows if len(r) >= cfg.min_len]
    return docs, vocab


def diagnose(cfg: DiagnoseConfig) -> dict:
    device = torch.device(cfg.device if torch.cuda.is_available() else "cpu")
    print(f"Model: {cfg.model}  precision: {cfg.precision}  device: {device}  trials: {cfg.n_trials}")
    tokens_ok = diagnose_special_tokens(cfg.model)
    docs, vocab = _load_docs(cfg)
    print(f"Documents: {len(docs)} (lengths {cfg.min_len}-{cfg.max_len})")
    base = DTYPE_MAP[cfg.precision]
    kw = simple_parse_kwargs_string(cfg.model_kwargs)

    def fresh(dtype):
        m = load_model(cfg.model, dtype=dtype, device=device, **kw)
        m.eval()
        return m

    configs = [(f"precision={cfg.precision}", base, False, False)]
    if cfg.precision != "fp32":
        configs += [("--precision fp32 --use_tf32_matmuls", torch.float32, False, True),
                    (f"--force_math_sdp (precision={cfg.precision})", base, True, False),
                    ("--precision fp32 --use_tf32_matmuls --force_math_sdp", torch.float32, True, True),
                    ("--precision fp32 --force_math_sdp", torch.float32, True, False)]

    print("\nTesting: equal-length batching (no padding)")
    eq_min, eq_flagged = _summarise(_trials(fresh(base), docs, cfg.n_trials, cfg.seed, device, vocab=vocab), cfg.threshold)

    results, passing = {}, None
    for label, dtype, math_sdp, tf32 in configs:
        print(f"\nTesting: {label}")
        if torch.cuda.is_available():
            torch.backends.cuda.enable_flash_sdp(not math_sdp)
            torch.backends.cuda.enable_mem_efficient_sdp(not math_sdp)
        torch.set_float32_matmul_precision("high" if tf32 else "highest")
        mn, flagged = _summarise(_trials(fresh(dtype), docs, cfg.n_trials, cfg.seed, device), cfg.threshold)
        results[label] = (flagged, mn)
        if flagged == 0:
            passing = label
            break

    print(f"\nReport for {cfg.model} ({cfg.n_trials} trials per configuration)")
    print(f"  {'PASS' if tokens_ok else 'FAIL'}  Special token check")
    print(f"  {'PASS' if eq_flagged == 0 else 'FAIL'}  Equal-length batching (min cos_sim={eq_min:.6f})")
    for label, (flagged, mn) in results.items():
        print(f"  {'PASS' if flagged == 0 else 'FAIL'}  {label}  (min cos_sim={mn:.6f})")
    first = next(iter(results))
    if results[first][0] == 0:
        print("RESULT: Gradients are consistent with default settings. No special flags needed.")
    elif passing is not None:
        print(f"RESULT: Gradients require non-default settings for consistency. Minimum required: {passing}")
    else:
        print("RESULT: No tested configuration produced consistent gradients.")
    return {"special_tokens_ok": tokens_ok, "equal_length_min_cos": eq_min, "configs": results, "passing": passing}
