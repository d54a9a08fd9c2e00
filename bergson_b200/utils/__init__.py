from .math import weighted_causal_lm_ce
from .utils import assert_type, get_layer_list

__all__ = ["assert_type", "get_layer_list", "weighted_causal_lm_ce"]
