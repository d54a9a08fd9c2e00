"""``collect_gradients``: one pass over the data with a ``GradientCollector`` attached
(reference ``bergson/collection.py:11-45``)."""

from __future__ import annotations

from .collector.collector import CollectorComputer
from .collector.gradient_collectors import GradientCollector
from .config.config import AttentionConfig, IndexConfig, PreprocessConfig
from .gradients import GradientProcessor
from .score.scorer import Scorer


def collect_gradients(
    model,
    data,
    processor: GradientProcessor,
    cfg: IndexConfig,
    *,
    batches: list[list[int]] | None = None,
    target_modules: set[str] | None = None,
    attention_cfgs: dict[str, AttentionConfig] | None = None,
    scorer: Scorer | None = None,
    preprocess_cfg: PreprocessConfig | None = None,
):
    collector = GradientCollector(
        model=model.base_model,
        cfg=cfg,
        processor=processor,
        target_modules=target_modules,
        data=data,
        scorer=scorer,
        preprocess_cfg=preprocess_cfg or PreprocessConfig(),
        attention_cfgs=attention_cfgs or {},
        filter_modules=cfg.filter_modules,
    )
    computer = CollectorComputer(model=model, data=data, collector=collector, batches=batches, cfg=cfg)
    computer.run_with_collector_hooks(desc="New worker - Collecting gradients")
    return collector
