"""``MagicConfig`` under the module path the reference uses
(``bergson/magic/config.py:7``); the class itself lives with the other configs."""

from ..config.config import MagicConfig

__all__ = ["MagicConfig"]
