from .omni_moe import OmniMoE, OmniMoEConfig

__all__ = ["OmniMoE", "OmniMoEConfig"]
