from ue5m3_fp4.nn.convert import (ConversionRecord, ProductPlan, convert_linear_modules, exclude_lm_head,
                                  plan_fp4_products, reserve_device_workspace, select_all_linears)
from ue5m3_fp4.nn.linear import LinearBackend, UE5M3Linear

__all__ = [
    "ConversionRecord",
    "LinearBackend",
    "ProductPlan",
    "UE5M3Linear",
    "plan_fp4_products",
    "reserve_device_workspace",
    "convert_linear_modules",
    "exclude_lm_head",
    "select_all_linears",
]
