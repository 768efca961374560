"""B200-native (sm_100a) FP8 paged-KV attention and Gated-DeltaNet recurrent kernels behind the
``green_attention`` SGLang plugin interface."""

__version__ = "0.1.0"
