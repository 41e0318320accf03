"""B200-native (sm_100a) decode / speculative-verify hot path behind the reference bundle's
`model.layers.*` and `logits_processor` operator interface.  All computation lives in
libb200nodes.so (hand-written CUDA, C ABI in include/b200nodes.h); this package is the host side."""
__version__ = "0.1.0"
