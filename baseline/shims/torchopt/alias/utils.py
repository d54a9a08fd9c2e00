from ..transform import scale_by_neg_lr


def _get_use_chain_flat() -> bool:
    return False


__all__ = ["_get_use_chain_flat", "scale_by_neg_lr"]
