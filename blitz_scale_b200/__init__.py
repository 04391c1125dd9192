"""blitz_scale_b200: a Blackwell-native (sm_100a) LLM serving framework with live autoscaling.

Layout: ``csrc`` native sources (CUDA kernels, C++ runtime / router / simulator cores), ``ops`` kernel
entry points, ``models`` shape registry + oracle + fused forward, ``runtime`` the per-GPU engine,
``parallel`` peer-memory data paths (parameter multicast, KV push, activation mailbox, TP fused
GEMMs), ``worker`` the gRPC service, ``router`` the orchestrator shells, ``sim`` trace replay and
stub workers, ``pb`` the wire contract.
"""
__version__ = "0.1.0"
