"""rptc_b200: host side of the B200-native RPTC decode / fused dequant-matmul library."""
from ._lib import (CODE_HASH, CODE_LITE, CODE_LUT, LAYOUT_CHUNKED, LAYOUT_ROWMAJOR, LAYOUT_TILED, LAYOUT_UNITMAJOR, QUIRK_K1_LANE0_SEED,
                   QUIRK_K2_LANE0_CARRY, QUIRK_NONE, XORDER_K2_LEGACY, XORDER_NATURAL, Format, RPTCError, lib)
from . import ops

__all__ = ["CODE_HASH", "CODE_LITE", "CODE_LUT", "LAYOUT_CHUNKED", "LAYOUT_ROWMAJOR", "LAYOUT_TILED", "LAYOUT_UNITMAJOR",
           "QUIRK_K1_LANE0_SEED", "QUIRK_K2_LANE0_CARRY", "QUIRK_NONE", "XORDER_K2_LEGACY", "XORDER_NATURAL", "Format",
           "RPTCError", "lib", "ops"]
