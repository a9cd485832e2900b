"""Storage format constants of the tiered KV cache.

Group-asymmetric quantization (reference: ``echokv_vllm/quant.py``): every
group stores an fp16 ``scale = (max - min) / (2**b - 1)`` (clamped to the
smallest normal fp16) and an fp16 ``min``; a code is
``round_half_even((x - min) / scale)`` clamped to ``[0, 2**b - 1]`` and a value
reads back as ``code * scale + min``.  ``scale`` and ``min`` are rounded to fp16
*before* the codes are computed.  V groups run along head_dim within a token;
K groups run over ``k_group`` consecutive tokens per channel.  Sub-byte codes
are packed little-endian: element ``i`` of a byte sits at bits
``[i * b, (i + 1) * b)``.

The arithmetic itself lives in the CUDA kernels (``csrc/common.cuh``:
``group_stats`` / ``quant_code``); this module only carries the constants the
host code needs.
"""

SUPPORTED_BITS = (2, 4, 8)

# Extra pool chunks a block of each tier needs beyond chunk 0 of its own page.
EXTRA_CHUNKS = {2: 0, 4: 1, 8: 3}
