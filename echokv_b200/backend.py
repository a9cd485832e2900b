"""vLLM attention backend over the B200 kernels (mixed-precision paged KV cache).

Same classes, methods, arguments and error behaviour as the reference's
``echokv_vllm/backend.py`` (backend class :72-118, metadata :121-141, builder :232-496, impl
:499-636), so vLLM drives it the same way:

* ``EchoKVAttentionBackend.customize_spec`` declares the page as one opaque byte state per token,
  sized for ``ECHOKV_MEM_BITS``; vLLM's cache manager then budgets exactly the bytes the store uses.
* ``EchoKVMetadataBuilder.build`` does all host work once per step for every layer of the group
  (``GroupRunner.plan_step``: write plan, block opening at each layer's tier, one metadata upload)
  and runs the canary for all layers one step after a fire.
* ``EchoKVAttentionImpl.do_kv_cache_update`` / ``forward`` only launch kernels on device metadata,
  so decode-only batches replay as full CUDA graphs.

There is no PyTorch or CPU path: tensors that are not on a CUDA device are rejected by the
kernel launchers.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from typing import ClassVar

import numpy as np
import torch

from vllm.forward_context import get_forward_context
from vllm.v1.attention.backend import (
    AttentionBackend,
    AttentionCGSupport,
    AttentionImpl,
    AttentionMetadataBuilder,
    AttentionType,
    MultipleOf,
)

from echokv_b200.config import load_config
from echokv_b200.controller import LayerController
from echokv_b200.host_slots import host_lens_and_slots, is_dummy_step
from echokv_b200.kernels.decode import decode_attention
from echokv_b200.kernels.write import gather_rows
from echokv_b200.kernels.prefill import ROW_PATH_MAX_CHUNK, build_dense, build_rows, prefill_attention
from echokv_b200.step import GroupRunner, StepMeta
from echokv_b200.tiered_cache import TieredLayout
from echokv_b200.write_plan import WriteMeta


class EchoKVAttentionBackend(AttentionBackend):
    forward_includes_kv_cache_update: bool = False
    supported_dtypes: ClassVar[list[torch.dtype]] = [torch.float16, torch.bfloat16, torch.float32]
    supported_kv_cache_dtypes: ClassVar[list[str]] = ["auto", "float16", "bfloat16"]

    @classmethod
    def customize_spec(cls, spec):
        if spec.head_size_v != spec.head_size:
            raise NotImplementedError("EchoKV requires head_size_v == head_size")
        cfg = load_config()
        nbytes = TieredLayout.per_token_bytes(spec.num_kv_heads, spec.head_size, cfg.mem_bits, cfg.k_group, cfg.v_group)
        return replace(spec, num_head_slots=1, state_content_bytes=nbytes)

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto"):
        """Shape (in elements of the model dtype) of a layer's slice of the pool on vLLM releases without
        ``customize_spec``: one opaque run of bytes per token, ``vllm_compat.slot_bytes`` per KV head."""
        from echokv_b200.vllm_compat import slot_bytes

        elt = torch.empty((), dtype=_model_dtype()).element_size()
        return (num_blocks, 1, block_size, num_kv_heads * slot_bytes(num_kv_heads, head_size) // elt)

    @staticmethod
    def get_supported_kernel_block_sizes(kv_cache_spec=None):
        return [MultipleOf(_block_multiple())]

    @classmethod
    def supports_block_size(cls, block_size) -> bool:
        return block_size is None or block_size % _block_multiple() == 0

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return head_size % 4 == 0 and head_size % load_config().v_group == 0

    @classmethod
    def supports_attn_type(cls, attn_type: str) -> bool:
        return attn_type == AttentionType.DECODER

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return EchoKVAttentionImpl

    @staticmethod
    def get_builder_cls():
        return EchoKVMetadataBuilder


@dataclass
class EchoKVMetadata:
    """One step's attention metadata, shared by every layer of the KV-cache group."""

    num_actual_tokens: int
    num_reqs: int
    query_start_loc_cpu: torch.Tensor
    seq_lens_cpu: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    write: WriteMeta | None = None  # None: no KV cache bound yet (memory profiling); attention is skipped
    canary_rows: torch.Tensor | None = None  # [canary_max_q] query rows to stash for the canary
    fire: bool = False  # this step's query rows feed the canary (measured at the next build)
    decode_rows: torch.Tensor | None = None  # [nd] query rows of single-token requests
    decode_reqs: torch.Tensor | None = None  # [nd] their block-table rows
    decode_lens: torch.Tensor | None = None  # [nd] their cache lengths (0 = CUDA-graph padding)
    num_splits: int = 1  # fixed decode split grid, so a graph can replay it
    split_floor: int = 1  # smallest number of blocks per decode split
    bps_dev: torch.Tensor | None = None  # blocks per decode split chosen for this step (read by the kernels at run time)
    prefill: list = field(default_factory=list)  # (q_start, q_end, ctx, dense_start) per chunk
    prefill_reqs: list = field(default_factory=list)  # block-table row of each chunk
    prefill_rows: tuple | None = None  # row path: per query token (row, request, causal limit), max limit
    prefill_dense: tuple | None = None  # dense path: dequant work list + varlen attention inputs


def split_batch(starts: np.ndarray, lens: np.ndarray, num_tokens: int):
    """Sort a step's requests into decode entries and prefill chunks (all numpy, no device work).

    Returns ``(decode_rows, decode_reqs, decode_lens, prefill, prefill_reqs, last_rows, last_ctx)``.
    A batch of single-token requests keeps one decode entry per request, padding included with
    length 0, which is the shape a CUDA graph replays; mixed batches keep live requests only.
    Reference: backend.py:369-391.
    """
    qlen = np.diff(starts)
    live = (qlen > 0) & (lens > 0)
    single = qlen == 1
    dec = np.arange(qlen.size) if (qlen <= 1).all() else np.flatnonzero(live & single)
    dec_lens = np.where(single[dec], lens[dec], 0)
    dec_rows = np.minimum(starts[:-1][dec], max(num_tokens - 1, 0))
    prefill, reqs, at = [], [], 0
    for r in np.flatnonzero(live & (qlen > 1)).tolist():
        ctx = int(lens[r])
        prefill.append((int(starts[r]), int(starts[r + 1]), ctx, at))
        reqs.append(r)
        at += ctx
    return dec_rows, dec, dec_lens, prefill, reqs, (starts[1:] - 1)[live], lens[live]


class CanarySchedule:
    """When the canary fires, and which measurement the controllers have not consumed yet.

    A fire step stashes query rows; the KL is measured at the next build (before that step's plan
    moves the K_ref ring) and fed to the controllers one measurement later, when it has long
    finished on the GPU, so reading it back does not stall the stream (reference:
    backend.py:314-333, 401-418).
    """

    def __init__(self, interval: int, max_q: int) -> None:
        self.interval, self.max_q = interval, max_q
        self.steps = 0
        self.armed = False
        self.stashed: tuple[int, float] | None = None  # (rows, mean context) of the last fire
        self.unread: tuple[torch.Tensor, float] | None = None  # finished KL [layers, tiers], its mean context

    def reset(self) -> None:
        self.stashed = self.unread = None

    def measure(self, runner: GroupRunner, tp_group=None) -> None:
        nq, ctx = self.stashed
        self.stashed = None
        if self.unread is not None:
            runner.observe(*self.unread)
            self.unread = None
        deltas = runner.measure_canary(nq, tp_group)
        if deltas is not None:
            self.unread = (deltas, ctx)

    def rows_for(self, dummy: bool, last_rows: np.ndarray, last_ctx: np.ndarray) -> tuple[np.ndarray, bool]:
        if not dummy:
            self.steps += 1
            self.armed = self.armed or self.steps % self.interval == 0
        rows = np.zeros(self.max_q, dtype=np.int64)
        if not (self.armed and last_rows.size):
            return rows, False
        self.armed = False
        k = min(self.max_q, last_rows.size)
        rows[:k] = last_rows[:k]
        self.stashed = (k, float(last_ctx[:k].mean()))
        return rows, True


class EchoKVMetadataBuilder(AttentionMetadataBuilder[EchoKVMetadata]):
    _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    @classmethod
    def get_cudagraph_support(cls, vllm_config, kv_cache_spec) -> AttentionCGSupport:
        # ECHOKV_CUDAGRAPH=0 makes attention run eagerly; the kernels handle any block size that is
        # a multiple of the K group, so nothing else rules graphs out.
        if os.environ.get("ECHOKV_CUDAGRAPH", "1") != "1":
            return AttentionCGSupport.NEVER
        return cls._cudagraph_support

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device) -> None:
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self.cfg = cfg = load_config()
        self.num_q_heads = _query_heads(vllm_config, layer_names)
        self.gqa = self.num_q_heads // kv_cache_spec.num_kv_heads
        # Exact CPU sequence lengths are needed for the host slot mapping; async speculative decoding
        # does not provide them.
        self.host_slots = vllm_config.speculative_config is None
        self.check_host_slots = os.environ.get("ECHOKV_CHECK_HOST_SLOTS", "0") == "1"
        self.host_slot_steps = 0
        self.residual_slots = _residual_slots(cfg, vllm_config)
        self.cap = getattr(vllm_config.compilation_config, "max_cudagraph_capture_size", None) or 512
        self.max_model_len = vllm_config.model_config.max_model_len
        self.runner: GroupRunner | None = None
        self.canary = CanarySchedule(cfg.canary_interval, cfg.canary_max_q)
        self._layers: list | None = None
        self._impls: list[EchoKVAttentionImpl] = []
        self._bound_ptr: int | None = None

    @property
    def num_splits(self) -> int:
        return self.runner.num_splits if self.runner is not None else 1

    # -- binding ------------------------------------------------------------------------------
    def _attach(self) -> bool:
        """Bind every layer of the group to its KV cache; False while vLLM has allocated none."""
        if self._layers is None:
            from vllm.config import get_layers_from_vllm_config
            from vllm.model_executor.layers.attention_layer_base import AttentionLayerBase

            self._layers = list(get_layers_from_vllm_config(self.vllm_config, AttentionLayerBase, self.layer_names).values())
        caches = [getattr(layer, "kv_cache", None) for layer in self._layers]
        if not caches or any(c is None or c.numel() == 0 for c in caches):
            return False
        if self._bound_ptr == caches[0].data_ptr():
            return True
        self._impls = [layer.impl for layer in self._layers]
        self.runner = bind_group(self._impls, caches, self.cfg, self.kv_cache_spec.block_size, self.residual_slots,
                                 self.cap, self.max_model_len)
        self._bound_ptr = caches[0].data_ptr()
        self.canary.reset()
        return True

    # -- build --------------------------------------------------------------------------------
    def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False) -> EchoKVMetadata:
        cm = common_attn_metadata
        if cm.causal is not True:
            raise NotImplementedError("EchoKV supports causal decoder attention only")
        n, t = cm.num_reqs, cm.num_actual_tokens
        dummy = is_dummy_step(cm)
        lens_cpu, slots_cpu = self._lens_and_slots(cm, n, t, dummy)
        starts = cm.query_start_loc_cpu[: n + 1].numpy().astype(np.int64)
        d_rows, d_reqs, d_lens, prefill, p_reqs, last_rows, last_ctx = split_batch(
            starts, lens_cpu.numpy().astype(np.int64), t)
        md = EchoKVMetadata(
            num_actual_tokens=t, num_reqs=n, query_start_loc_cpu=cm.query_start_loc_cpu[: n + 1].cpu(),
            seq_lens_cpu=lens_cpu, block_table=cm.block_table_tensor, slot_mapping=cm.slot_mapping,
            prefill=prefill, prefill_reqs=p_reqs)
        if self._attach():
            if self.canary.stashed is not None:
                self.canary.measure(self.runner, _tp_group())
            rows, md.fire = self.canary.rows_for(dummy, last_rows, last_ctx)
            step: StepMeta = self.runner.plan_step(slots_cpu, decode=(d_rows, d_reqs, d_lens), canary=rows)
            md.write, md.canary_rows, md.num_splits = step.write, step.canary_rows, step.num_splits
            md.split_floor, md.bps_dev = self.runner.split_floor, step.bps_dev
            md.decode_rows, md.decode_reqs, md.decode_lens = step.decode_rows, step.decode_reqs, step.decode_lens
        if prefill:
            if max(qe - qs for qs, qe, _, _ in prefill) <= ROW_PATH_MAX_CHUNK:
                md.prefill_rows = build_rows(prefill, p_reqs, self.device)
            else:
                md.prefill_dense = build_dense(prefill, p_reqs, self.kv_cache_spec.block_size, self.device)
        return md

    def _lens_and_slots(self, cm, n: int, t: int, dummy: bool):
        host = host_lens_and_slots(cm, self.kv_cache_spec.block_size) if self.host_slots else None
        if host is not None:
            self.host_slot_steps += 1
            if not self.check_host_slots:
                return host
        elif self.check_host_slots and self.host_slots and not dummy:
            raise AssertionError("ECHOKV_CHECK_HOST_SLOTS=1 but the host slot mapping is unavailable")
        # Device-to-host copies wait for the stream to drain; only dummy steps and checks take them.
        dev = cm.seq_lens[:n].cpu(), cm.slot_mapping[:t].cpu()
        if host is not None and not (torch.equal(host[0], dev[0].long()) and torch.equal(host[1], dev[1].long())):
            raise AssertionError("EchoKV host slot mapping differs from vLLM's")
        return dev


def bind_group(impls, caches, cfg, block_size: int, residual_slots: int, cap: int, max_model_len: int) -> GroupRunner:
    """One ``GroupRunner`` over the layers' cache slices and the buffers their impls allocated."""
    first = impls[0]
    layout = TieredLayout(num_kv_heads=first.num_kv_heads, head_size=first.head_size, block_size=block_size,
                          mem_bits=cfg.mem_bits, k_group=cfg.k_group, v_group=cfg.v_group)
    pages = [page_view(c, block_size) for c in caches]
    dev = pages[0].device
    for impl in impls:
        impl.residual, impl.kref_buf, impl.stash = impl.residual.to(dev), impl.kref_buf.to(dev), impl.stash.to(dev)
    runner = GroupRunner(
        layout, pages, first.num_heads, first.scale, [i.controller for i in impls], residual_slots,
        first.residual.dtype, kref_window=cfg.kref_window, canary_max_q=cfg.canary_max_q, cap=cap,
        max_model_len=max_model_len, residuals=[i.residual for i in impls], krefs=[i.kref_buf for i in impls],
        stashes=[i.stash for i in impls])
    for k, impl in enumerate(impls):
        impl.runner, impl.index, impl.store = runner, k, runner.stores[k]
    return runner


def page_view(kv_cache: torch.Tensor, block_size: int) -> torch.Tensor:
    """A layer's slice of vLLM's pool as ``[num_blocks, block_size * bytes_per_token]`` bytes; the block
    stride may exceed the page (pools that interleave layers)."""
    raw = kv_cache.view(torch.uint8)
    if raw.dim() != 4 or raw.shape[1] != 1 or raw.shape[2] != block_size or raw.stride(3) != 1 or raw.stride(2) != raw.shape[3]:
        raise RuntimeError(f"unexpected EchoKV cache view shape={tuple(raw.shape)} stride={raw.stride()}")
    return torch.as_strided(raw, (raw.shape[0], block_size * raw.shape[3]), (raw.stride(0), 1))


class EchoKVAttentionImpl(AttentionImpl[EchoKVMetadata]):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int | None = None,
                 alibi_slopes=None, sliding_window=None, kv_cache_dtype: str = "auto", logits_soft_cap=None,
                 attn_type: str = AttentionType.DECODER, kv_sharing_target_layer_name=None, sinks=None) -> None:
        refused = [what for what, on in (
            ("alibi", alibi_slopes is not None), ("sliding window", sliding_window is not None),
            ("logits soft cap", bool(logits_soft_cap)), ("attention sinks", sinks is not None),
            ("KV sharing", kv_sharing_target_layer_name is not None),
            (f"attn_type={attn_type}", attn_type != AttentionType.DECODER)) if on]
        if refused:
            raise NotImplementedError(f"EchoKV does not support: {', '.join(refused)}")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads or num_heads
        self.kv_cache_dtype = kv_cache_dtype
        self.cfg = cfg = load_config()
        self.controller = LayerController(cfg.controller)
        # Allocated during model construction so vLLM's memory profiler counts them: full-precision K
        # of each block's open group (+1 spare row), the K_ref ring, the canary's stashed query rows.
        dt = _model_dtype()
        self.residual = torch.zeros(_residual_slots(cfg) + 1, cfg.k_group, self.num_kv_heads, head_size, dtype=dt)
        self.kref_buf = torch.zeros(cfg.kref_window, self.num_kv_heads, head_size, dtype=torch.float32)
        self.stash = torch.zeros(cfg.canary_max_q, num_heads, head_size, dtype=dt)
        self.runner: GroupRunner | None = None
        self.index = 0
        self.store = None
        self.forward_calls = 0  # eager forwards; graph replays do not enter Python

    def bind(self, kv_cache: torch.Tensor, shared=None) -> None:
        """Wrap ``kv_cache`` in a store of its own (a group of one layer)."""
        bind_group([self], [kv_cache], self.cfg, kv_cache.shape[2], self.residual.shape[0] - 1, 512, 8192)

    def do_kv_cache_update(self, layer, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                           slot_mapping: torch.Tensor) -> None:
        md = _this_layer(get_forward_context().attn_metadata, layer)
        if md is None or md.write is None:
            return
        self.store.apply(md.write, key, value, self.kref_buf, capturing=_capturing(key))

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                attn_metadata: EchoKVMetadata, output: torch.Tensor, output_scale=None, output_block_scale=None):
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantization is not supported by EchoKV")
        md = attn_metadata
        if md is None or md.write is None:  # profiling / warmup run
            return output
        self.forward_calls += 1
        if md.prefill:
            prefill_attention(self.store, query, output, md.prefill, md.prefill_reqs, md.block_table, self.scale,
                              dense=md.prefill_dense, rows=md.prefill_rows)
        if md.decode_rows is not None:
            decode_attention(self.store, query, md.block_table, md.decode_lens, self.scale, md.split_floor,
                             q_rows=md.decode_rows, bt_rows=md.decode_reqs,
                             out=output.view(output.shape[0], -1, query.shape[-1]), num_splits=md.num_splits,
                             bps_dev=md.bps_dev)
        # A graph captures the copy unconditionally: its row indices are valid either way.
        if md.fire or _capturing(query):
            gather_rows(query, md.canary_rows, self.stash)
        return output


def _this_layer(md, layer):
    if isinstance(md, list):  # speculative decoding: entry 0 is the base model
        md = md[0]
    return md[layer.layer_name] if isinstance(md, dict) else md


def _capturing(t: torch.Tensor) -> bool:
    return t.is_cuda and torch.cuda.is_current_stream_capturing()


def _block_multiple() -> int:
    return max(16, load_config().k_group)


def _query_heads(vllm_config, layer_names) -> int:
    try:
        from vllm.v1.attention.backends.utils import get_num_attention_heads_from_layers

        n = get_num_attention_heads_from_layers(vllm_config, layer_names)
        if n:
            return n
    except ImportError:
        pass
    return vllm_config.model_config.get_num_attention_heads(vllm_config.parallel_config)


def _current_vllm_config():
    try:
        from vllm.config import get_current_vllm_config_or_none

        return get_current_vllm_config_or_none()
    except ImportError:
        return None


def _residual_slots(cfg, vllm_config=None) -> int:
    if cfg.residual_slots is not None:
        return cfg.residual_slots
    vc = vllm_config if vllm_config is not None else _current_vllm_config()
    return (vc.scheduler_config.max_num_seqs if vc is not None else 256) + 16


def _model_dtype() -> torch.dtype:
    vc = _current_vllm_config()
    return vc.model_config.dtype if vc is not None else torch.float32


def _tp_group():
    """The tensor-parallel process group (None when there is one rank): each rank's canary sees only
    its own KV heads, so the KL is averaged before the controllers tick (reference: backend.py:665-675)."""
    try:
        from vllm.distributed import get_tensor_model_parallel_world_size, get_tp_group
    except ImportError:
        return None
    try:
        if get_tensor_model_parallel_world_size() == 1:
            return None
        return get_tp_group().device_group
    except AssertionError:  # no model-parallel state (unit tests)
        return None
