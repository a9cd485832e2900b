"""Bridges to vLLM releases older than the one the reference plugin targets (0.32).

The reference declares its page size through ``AttentionBackend.customize_spec`` (backend.py:82-90 of the
reference), a hook that vLLM 0.22 does not have.  There the page size comes from the KV-cache spec an attention
layer builds for itself, and the one spec whose page is *not* ``2 * block * heads * head_size * dtype`` is
``TQFullAttentionSpec`` (page = block_size * num_kv_heads * tq_slot_size bytes).  ``install()`` makes the layers
served by this package's backend return that spec with a slot sized for ``ECHOKV_MEM_BITS``, so vLLM's cache
manager budgets the bytes the tiered store really uses (and reports the larger token capacity).
"""

from __future__ import annotations

from echokv_b200.config import load_config
from echokv_b200.tiered_cache import TieredLayout


def slot_bytes(num_kv_heads: int, head_size: int) -> int:
    """Bytes per (token, KV head) of the page vLLM allocates: the store's bytes per token split evenly over the
    heads, rounded up to a multiple of 4 so that the page is a whole number of elements of any model dtype."""
    cfg = load_config()
    per_token = TieredLayout.per_token_bytes(num_kv_heads, head_size, cfg.mem_bits, cfg.k_group, cfg.v_group)
    per_head = -(-per_token // num_kv_heads)
    return -(-per_head // 4) * 4


def needs_spec_patch() -> bool:
    from vllm.v1.attention.backend import AttentionBackend

    return not hasattr(AttentionBackend, "customize_spec")


def install() -> bool:
    """Patch ``Attention.get_kv_cache_spec`` once; True if this vLLM needed it."""
    if not needs_spec_patch():
        return False
    from vllm.model_executor.layers.attention.attention import Attention
    from vllm.v1.kv_cache_interface import FullAttentionSpec, TQFullAttentionSpec

    if getattr(Attention.get_kv_cache_spec, "_echokv", False):
        return True
    original = Attention.get_kv_cache_spec

    def get_kv_cache_spec(self, vllm_config):
        spec = original(self, vllm_config)
        backend = self.get_attn_backend()
        ours = getattr(backend, "__module__", "").startswith("echokv_b200")
        if not ours or type(spec) is not FullAttentionSpec:
            return spec
        return TQFullAttentionSpec(
            block_size=spec.block_size, num_kv_heads=spec.num_kv_heads, head_size=spec.head_size,
            head_size_v=spec.head_size_v, dtype=spec.dtype,
            tq_slot_size=slot_bytes(spec.num_kv_heads, spec.head_size))

    get_kv_cache_spec._echokv = True
    Attention.get_kv_cache_spec = get_kv_cache_spec
    return True
