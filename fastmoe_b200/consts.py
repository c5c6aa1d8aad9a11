"""Implementation selector of the MoE layer: the two members and string values that
polkadot21/fastmoe callers pass (src/fastmoe/consts.py:4-6), `MoEImplementation.FAST` for the
no-cat combine and `MoEImplementation.STANDARD` for cat + index_add_."""

import enum

MoEImplementation = enum.StrEnum(
    "MoEImplementation",
    {"FAST": "fast", "STANDARD": "standard"},
    module=__name__,
)
