"""Normalisers from optimizer checkpoints: index -> parameter mapping for one and two
parameter groups, tied weights, transposed (Conv1D) layers, factored and quantised states,
bias moments, module filters and the error cases."""

import pytest
import torch
import torch.nn as nn

from bergson_b200.gradients import AdafactorNormalizer, AdamNormalizer
from bergson_b200.models.common import Conv1D
from bergson_b200.utils.load_from_optimizer import (
    load_from_optimizer, load_optimizer, optimizer_param_index_to_name, orient_second_moment,
    save_second_moments_as_optimizer_pt)


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(10, 4)
        self.norm = nn.LayerNorm(4)
        self.a = nn.Linear(4, 6, bias=True)
        self.b = nn.Linear(6, 8, bias=False)
        self.head = nn.Linear(4, 10, bias=False)
        self.head.weight = self.emb.weight  # tied, as in GPT-2

    def forward(self, ids):
        h = self.norm(self.emb(ids))
        return self.head(h) + self.b(self.a(h)).sum(-1, keepdim=True)


def _trained_optimizer(model, groups=None, steps=2):
    opt = torch.optim.AdamW(groups or model.parameters(), lr=1e-2)
    for _ in range(steps):
        opt.zero_grad()
        model(torch.arange(6)[None]).square().mean().backward()
        opt.step()
    return opt


def test_single_group_follows_named_parameters_order(tmp_path):
    torch.manual_seed(0)
    model = Block()
    opt = _trained_optimizer(model)
    torch.save(opt.state_dict(), tmp_path / "optimizer.pt")
    names = [n for n, _ in model.named_parameters()]
    assert "head.weight" not in names  # the tied duplicate is dropped
    sd = load_optimizer(str(tmp_path))  # a directory resolves to its optimizer.pt
    assert optimizer_param_index_to_name(sd, model) == dict(enumerate(names))
    norms = load_from_optimizer(model, str(tmp_path / "optimizer.pt"), include_bias=True)
    assert set(norms) == {"emb", "a", "b"}  # 2-D weights only; the tied head goes by its surviving name
    idx = names.index("a.weight")
    torch.testing.assert_close(norms["a"].weight_avg_sq, opt.state_dict()["state"][idx]["exp_avg_sq"])
    torch.testing.assert_close(norms["a"].bias_avg_sq, opt.state_dict()["state"][names.index("a.bias")]["exp_avg_sq"])
    assert norms["b"].bias_avg_sq is None
    assert load_from_optimizer(model, str(tmp_path), include_bias=False)["a"].bias_avg_sq is None
    assert set(load_from_optimizer(model, str(tmp_path), target_modules={"b"})) == {"b"}


def test_two_groups_are_the_decay_and_no_decay_split(tmp_path):
    """The Hugging Face trainer puts weights first and norm parameters and biases second."""
    torch.manual_seed(0)
    model = Block()
    named = dict(model.named_parameters())
    decay = [n for n in named if "norm" not in n and "bias" not in n]
    no_decay = [n for n in named if n not in decay]
    opt = _trained_optimizer(model, [{"params": [named[n] for n in decay], "weight_decay": 0.1},
                                     {"params": [named[n] for n in no_decay], "weight_decay": 0.0}])
    sd = opt.state_dict()
    mapping = optimizer_param_index_to_name(sd, model)
    assert [mapping[i] for i in range(len(named))] == decay + no_decay
    torch.save(sd, tmp_path / "optimizer.pt")
    norms = load_from_optimizer(model, str(tmp_path), include_bias=True)
    torch.testing.assert_close(norms["b"].weight_avg_sq, sd["state"][decay.index("b.weight")]["exp_avg_sq"])
    torch.testing.assert_close(norms["a"].bias_avg_sq, sd["state"][len(decay) + no_decay.index("a.bias")]["exp_avg_sq"])
    # a split that does not fit the model is refused rather than guessed
    sd["param_groups"][0]["params"] = sd["param_groups"][0]["params"][:-1]
    with pytest.raises(ValueError, match="param groups"):
        optimizer_param_index_to_name(sd, model)


def test_a_layout_that_does_not_fit_is_detected(tmp_path):
    model = Block()
    sd = _trained_optimizer(model).state_dict()
    sd["state"][1], sd["state"][3] = sd["state"][3], sd["state"][1]  # entries of different shapes swapped
    with pytest.raises(ValueError, match="second-moment shape"):
        optimizer_param_index_to_name(sd, model)


def test_export_names_survive_tied_weights(tmp_path):
    model = Block()
    params = dict(model.named_parameters())
    marks = {n: float(1000 + i) for i, n in enumerate(sorted(params))}
    state = {"nu": {n: torch.full_like(p, marks[n]) for n, p in params.items()}}
    n = save_second_moments_as_optimizer_pt(model, state, tmp_path / "optimizer.pt")
    assert n == len(params)
    norms = load_from_optimizer(model, str(tmp_path))
    assert "emb" in norms and "head" not in norms
    for module, norm in norms.items():
        assert isinstance(norm, AdamNormalizer) and float(norm.weight_avg_sq.flatten()[0]) == marks[module + ".weight"]
    with pytest.raises(ValueError, match="nu"):
        save_second_moments_as_optimizer_pt(model, {"mu": {}}, tmp_path / "x.pt")


def test_transposed_layers_and_factored_states(tmp_path):
    model = nn.Sequential()
    model.c = Conv1D(6, 4)  # weight stored [in=4, out=6]
    model.fc = nn.Linear(4, 6)
    v = torch.rand(4, 6)
    row, col = torch.rand(4), torch.rand(6)  # factored over the stored [in, out] layout
    torch.save({"state": {0: {"exp_avg_sq": v, "param_name": "c.weight"},
                          1: {"exp_avg_sq_row": torch.rand(6), "exp_avg_sq_col": torch.rand(4), "param_name": "fc.weight"}},
                "param_groups": [{"params": [0, 1]}]}, tmp_path / "mixed.pt")
    norms = load_from_optimizer(model, str(tmp_path / "mixed.pt"))
    torch.testing.assert_close(norms["c"].weight_avg_sq, v.T)  # always [out, in]
    assert isinstance(norms["fc"], AdafactorNormalizer) and norms["fc"].row.shape == (6,) and norms["fc"].col.shape == (4,)
    torch.save({"state": {0: {"exp_avg_sq_row": row, "exp_avg_sq_col": col, "param_name": "c.weight"}},
                "param_groups": [{"params": [0]}]}, tmp_path / "fact_t.pt")
    got = load_from_optimizer(model, str(tmp_path / "fact_t.pt"))["c"]
    torch.testing.assert_close(got.row, col)
    torch.testing.assert_close(got.col, row)
    # 8-bit optimizers keep the second moment inside a quantisation record
    torch.save({"state": {0: {"__bnb_optimizer_quant_state__": {"state2": torch.rand(6, 4)}, "param_name": "fc.weight"}},
                "param_groups": [{"params": [0]}]}, tmp_path / "bnb.pt")
    assert isinstance(load_from_optimizer(model, str(tmp_path / "bnb.pt"))["fc"], AdamNormalizer)


def test_orient_second_moment():
    t = torch.rand(4, 6)
    assert orient_second_moment(t, 4, 6).shape == (4, 6) and orient_second_moment(t, 6, 4).shape == (6, 4)
    assert orient_second_moment(t, 5, 6) is None
    sq = torch.rand(4, 4)
    torch.testing.assert_close(orient_second_moment(sq, 4, 4, layer=Conv1D(4, 4)), sq.T)  # the layer type decides
    torch.testing.assert_close(orient_second_moment(sq, 4, 4, layer=nn.Linear(4, 4)), sq)


def test_missing_files_and_empty_states(tmp_path):
    with pytest.raises(FileNotFoundError, match="hf://"):
        load_optimizer(str(tmp_path / "nowhere"))
    model = nn.Sequential()
    model.fc = nn.Linear(4, 6)
    torch.save({"state": {0: {"momentum_buffer": torch.rand(6, 4)}}, "param_groups": [{"params": [0]}]}, tmp_path / "sgd.pt")
    with pytest.raises(AssertionError, match="No optimizer second moments"):
        load_from_optimizer(model, str(tmp_path / "sgd.pt"))


def test_entry_format_helpers():
    from bergson_b200.utils.load_from_optimizer import (
        OptimizerStateFormat, get_normalizers, get_optimizer_state_format, get_unfactored_second_moment)

    v = torch.rand(6, 4)
    assert get_optimizer_state_format({"exp_avg_sq": v}) is OptimizerStateFormat.UNFACTORED
    assert get_optimizer_state_format({"exp_avg_sq_row": torch.rand(6), "exp_avg_sq_col": torch.rand(4)}) is OptimizerStateFormat.FACTORED
    bnb = {"__bnb_optimizer_quant_state__": {"state2": v}}
    assert get_optimizer_state_format(bnb) is OptimizerStateFormat.UNFACTORED
    assert get_optimizer_state_format({"momentum_buffer": v}) is None and get_optimizer_state_format("nope") is None
    assert get_unfactored_second_moment({"exp_avg_sq": v}) is v and get_unfactored_second_moment(bnb) is v
    with pytest.raises(KeyError):
        get_unfactored_second_moment({"exp_avg_sq_row": torch.rand(6)})
    sd = {"state": {0: {"exp_avg_sq": v}, 1: {"exp_avg_sq": torch.rand(6)}, 2: {"exp_avg_sq": torch.rand(3, 6), "param_name": "model.out.weight"}}}
    names = {0: "model.fc.weight", 1: "model.fc.bias", 2: "ignored.by.param_name"}
    got = get_normalizers(sd, names, None, ".default", True, "cpu", base_prefix="model.")
    assert set(got) == {"fc.default", "out.default"}  # relative to the base model, adapter suffix appended
    torch.testing.assert_close(got["fc.default"].bias_avg_sq, sd["state"][1]["exp_avg_sq"])
    assert set(get_normalizers(sd, names, {"out.default"}, ".default", False, "cpu", base_prefix="model.")) == {"out.default"}
