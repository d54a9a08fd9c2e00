"""B200-native data attribution: gradient stores, TrackStar, (E)K-FAC / Shampoo
influence, SOURCE, MAGIC, with hand-written sm_100a kernels on the hot paths."""

__version__ = "0.1.0"

_LAZY = {
    "Builder": ".builder",
    "collect_gradients": ".collection",
    "CollectorComputer": ".collector.collector",
    "GradientCollector": ".collector.gradient_collectors",
    "InMemoryCollector": ".collector.in_memory_collector",
    "AttentionConfig": ".config.config",
    "DataConfig": ".config.config",
    "IndexConfig": ".config.config",
    "PreprocessConfig": ".config.config",
    "QueryConfig": ".config.config",
    "ScoreConfig": ".config.config",
    "FaissConfig": ".config.config",
    "ModuleGradients": ".data",
    "TokenGradients": ".data",
    "load_gradient_dataset": ".data",
    "load_gradients": ".data",
    "load_module_gradients": ".data",
    "load_token_gradients": ".data",
    "GradientProcessor": ".gradients",
    "mix_autocorrelation_matrices": ".process_grads",
    "Attributor": ".query.attributor",
    "Scorer": ".score.scorer",
    "FiniteDiff": ".utils.gradcheck",
    "load_from_optimizer": ".utils.load_from_optimizer",
}

__all__ = sorted(_LAZY) + ["__version__"]


def __getattr__(name: str):
    # Attribute access imports the defining module on first use, which keeps
    # ``import bergson_b200`` cheap for the CLI's ``--help``.
    if name in _LAZY:
        import importlib

        value = getattr(importlib.import_module(_LAZY[name], __name__), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
