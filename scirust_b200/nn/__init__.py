from .rng import PcgEngine, Philox4x32  # noqa: F401
from .init import KaimingNormal, XavierUniform, Zeros, SmallNormal, TruncatedNormal, Initializer  # noqa: F401
from .modules import (Module, Sequential, Linear, ReLU, Sigmoid, Tanh, GELU, SiLU, Dropout, Embedding, LayerNorm,  # noqa: F401
                      RMSNorm, BatchNorm1d, BatchNorm2d, Conv2d, ConvTranspose2d, MaxPool2d, GlobalAvgPool2d,
                      Padding, SinusoidalPositionalEncoding, rope_frequencies, yarn_frequencies)
from .loss import CrossEntropyLoss, MSELoss, NLLLoss, PoissonNLLLoss, PINNLoss, CTCLoss  # noqa: F401
from .transformer import (MultiHeadAttention, TransformerBlock, TransformerEncoder, TransformerDecoder, MoE,  # noqa: F401
                          MiniLLM, FeedForward, flash_attention_blockwise)
from .vision import ResidualBlock, ResNet, resnet18, resnet34, MnistCNN, CifarCNN, ViT  # noqa: F401
from .kv_cache import (AttentionBackend, PlainKvCache, PagedKvCache, QuantKvCache, ElasticKvCache, LatentKvCache,  # noqa: F401
                       TieredKvCache)
from .audio import AudioEncoder, ctc_loss  # noqa: F401
from .contracts import CertifiedModule, ValueBoundedContract  # noqa: F401
from .ensemble import DeepEnsemble  # noqa: F401
from .sampling import SamplingConfig, sample_token  # noqa: F401
