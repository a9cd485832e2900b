"""Entry point ``echokv`` of the ``vllm.general_plugins`` group.

vLLM imports and calls ``register()`` in the engine-core process and in every worker before it
builds a model.  With ``ECHOKV_ENABLE=1`` the call hooks the block tables (host slot mapping) and
puts this package's backend in the ``CUSTOM`` slot of vLLM's attention-backend registry; a model
then opts in with ``attention_config={"backend": "CUSTOM"}``.  Without the variable nothing is
touched.  Follows the reference's ``echokv_vllm/plugin.py:17-28``, minus its CPU-platform
override: these kernels run on CUDA devices only.
"""

from __future__ import annotations

import os

BACKEND_PATH = "echokv_b200.backend.EchoKVAttentionBackend"


def enabled() -> bool:
    return os.environ.get("ECHOKV_ENABLE", "0") == "1"


def register() -> None:
    if enabled():
        from vllm.v1.attention.backends import registry

        from echokv_b200 import host_slots, vllm_compat

        host_slots.install()
        vllm_compat.install()  # page size on vLLM releases without AttentionBackend.customize_spec
        registry.register_backend(registry.AttentionBackendEnum.CUSTOM, BACKEND_PATH)
