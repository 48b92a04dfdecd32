"""Training layer placeholder.

The reference exports ``MoEExpertLayer`` (``lightmoe/training.py``); this build
covers the inference path only, so the name resolves and refuses to construct.
"""


class MoEExpertLayer:
    def __init__(self, hidden_size, intermediate_size, num_experts, top_k, *args, **kwargs):
        raise NotImplementedError("MoEExpertLayer (training) is outside this inference-only build")


__all__ = ["MoEExpertLayer"]
