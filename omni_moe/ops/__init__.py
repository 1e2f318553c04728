from omni_moe_b200.ops import *  # noqa: F401,F403
