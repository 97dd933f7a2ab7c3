"""savanna_b200: B200-native pretraining framework for convolutional multi-hybrid models
(StripedHyena 2 / Evo 2 style: Hyena-SE, Hyena-MR, Hyena-LI and attention)."""
__version__ = "0.1.0"

from .config import GlobalConfig  # noqa: F401


def print_rank_0(*args, **kwargs):
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kwargs, flush=True)
