"""nanochat_b200: the KV-cache decode path of nanochat as hand-written sm_100a CUDA kernels
behind the reference's own Python interface (KVCache, flash_attn, the attention KV branch)."""
