"""Import target for TorchTitan's ``experimental.custom_import`` setting."""

from ue5m3_fp4.integrations.torchtitan.registration import register_torchtitan

register_torchtitan()
