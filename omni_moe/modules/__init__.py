from omni_moe_b200.modules.omni_moe import OmniMoE, OmniMoEConfig  # noqa: F401
