"""slopllm_b200: a B200 (sm_100a) inference engine for the glm_moe_dsa family and friends."""
__version__ = "0.1.0"
