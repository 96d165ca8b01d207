"""crosspool_b200 — Blackwell-native multi-model co-location serving with attention/FFN disaggregation.

Attention, KV cache and sampling run on *attention devices*; every decoder FFN (dense or MoE) lives
on a shared pool of *FFN devices*; a daemon control plane plans placement, brokers transport memory
and arbitrates elastic KV capacity. The data plane is hand-written sm_100a CUDA (tcgen05/TMEM GEMMs
fed by TMA, fused with their NVLink transfers).
"""

__version__ = "0.1.0"
