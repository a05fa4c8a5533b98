"""Layers of the framework (see modules.py, conv.py and transformer.py)."""
from .conv import BatchNorm, Conv2d, MaxPool2d
from .modules import (BatchNorm1d, Dropout, Embedding, Flatten, GELU, LayerNorm, Linear, ReLU, RMSNorm,
                      Sequential, Sigmoid, SiLU, Softmax, SwiGLU, Tanh)
from .transformer import (FeedForward, SelfAttention, TransformerBlock, TransformerConfig,
                          packed_attention)
