from .backbone import Backbone, build_model, param_groups
from .block import ParallelBlock
from .mixer import ParallelSequenceMixer, SelfAttention
from .hyena import CausalDepthwiseConv1d, HyenaOperator, ShortHyenaOperator
from .filters import ExplicitSingleDecayFilter, ImplicitModalFilter
from .norms import RMSNorm, LayerNorm, get_norm
from .mlp import ParallelGLU, ParallelMLP
from . import losses
