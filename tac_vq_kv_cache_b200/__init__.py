"""B200-native hard residual GSRQ/CQ KV-cache quantization: encode, code storage, attention over codes.

``jointkv``    reference-compatible operator API (codecs, functional quantizers, rate ledger)
``ops``        tensor-level calls into libtacvq.so (C ABI in include/tacvq.h)
``code_cache`` preallocated uint8 code store with in-place append and decode-step attention
``dist``       sharding helpers and the cross-GPU merge of partial softmax states
"""

__version__ = "0.1.0"
