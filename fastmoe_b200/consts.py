"""Implementation selector of the MoE layer, as in polkadot21/fastmoe (src/fastmoe/consts.py:4-6)."""

from enum import StrEnum


class MoEImplementation(StrEnum):
    FAST = "fast"
    STANDARD = "standard"
