from ue5m3_fp4.nn.convert import ConversionRecord, convert_linear_modules, exclude_lm_head, select_all_linears
from ue5m3_fp4.nn.linear import LinearBackend, UE5M3Linear

__all__ = [
    "ConversionRecord",
    "LinearBackend",
    "UE5M3Linear",
    "convert_linear_modules",
    "exclude_lm_head",
    "select_all_linears",
]
