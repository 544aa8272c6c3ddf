"""B200 (sm_100a) kernels for the sparse-attention selection path of TransArch:
lightning-indexer scoring, top-k selection, HISA / MISA variants, sparse MLA decode and the
key-sharded multi-GPU merge, behind the reference's own call signatures."""

__version__ = "0.1.0"
