"""Slot mapping and sequence lengths on the host, without a device-to-host copy.

vLLM computes ``slot_mapping`` on the GPU, so ``CommonAttentionMetadata`` only carries it as a
device tensor; the write planner needs it on the host and copying it back would wait for the
stream to drain (with async scheduling: the whole previous step).  Query positions follow from
``query_start_loc_cpu`` and ``seq_lens_cpu_upper_bound``; block ids come from a host mirror of the
block table.  Same role and hooks as the reference's ``echokv_vllm/host_slots.py``:

* V1 model runner (``BlockTable``): its CPU table ``block_table.np`` is the source of the GPU copy,
  indexed by batch row; every instance is remembered (``install`` :115-131, ``_wrap_init`` :42-54).
* V2 model runner (``BlockTables``): tables live on the GPU, indexed by request slot and written
  through ``append_block_ids``; those writes are mirrored in numpy and batch rows map to slots
  through ``cm.req_idx`` (``install_v2`` :61-84).

Dummy steps (warmup, profiling, CUDA-graph capture, idle data-parallel ranks) carry an all -1
slot mapping on the device while their block-table rows may belong to live requests; they are
detected and left to the device copy, so nothing is written where vLLM would not write.
"""

from __future__ import annotations

import weakref

import numpy as np
import torch

_MARK = "_echokv_b200_wrapped"
_v1_tables: "weakref.WeakSet" = weakref.WeakSet()
_v2_tables: "weakref.WeakSet" = weakref.WeakSet()
_v1_dummy_depth = 0  # > 0 while a V1 runner's _dummy_run is on the stack


def _already(fn) -> bool:
    return getattr(fn, _MARK, False)


def _tag(fn):
    setattr(fn, _MARK, True)
    return fn


def _remember_instances(cls, registry, after_init=None) -> None:
    """Wrap ``cls.__init__`` so every new instance lands in ``registry`` (once per class)."""
    init = cls.__init__
    if _already(init):
        return

    def __init__(self, *args, **kwargs):
        init(self, *args, **kwargs)
        if after_init is not None:
            after_init(self)
        registry.add(self)

    cls.__init__ = _tag(__init__)


def _flag_dummy(cls, method: str, dummy: bool) -> None:
    """Record on the instance whether its latest slot mapping is a dummy (all-PAD) one."""
    orig = getattr(cls, method)
    if _already(orig):
        return

    def wrapper(self, *args, **kwargs):
        self._echokv_dummy = dummy
        return orig(self, *args, **kwargs)

    setattr(cls, method, _tag(wrapper))


def install_v2(cls) -> None:
    """Mirror ``cls.append_block_ids`` on the host (V2 ``BlockTables``)."""

    def make_mirror(self) -> None:
        self._echokv_np = [np.zeros(tuple(t.gpu.shape), dtype=np.int64) for t in self.block_tables]

    _remember_instances(cls, _v2_tables, after_init=make_mirror)
    orig = cls.append_block_ids
    if not _already(orig):

        def append_block_ids(self, req_index, new_block_ids, overwrite):
            groups = range(self.num_kv_cache_groups)
            first = [0 if overwrite else int(self.num_blocks.np[g, req_index]) for g in groups]
            orig(self, req_index, new_block_ids, overwrite)
            to_null = getattr(self, "redirect_writes_to_null_block", False)
            for g in groups:
                ids = new_block_ids[g]
                self._echokv_np[g][req_index, first[g]: first[g] + len(ids)] = [0] * len(ids) if to_null else ids

        cls.append_block_ids = _tag(append_block_ids)
    _flag_dummy(cls, "compute_slot_mappings", False)
    _flag_dummy(cls, "get_dummy_slot_mappings", True)


def install_v1_dummy(cls) -> None:
    """Track ``cls._dummy_run`` (V1 model runner): its steps use the device copy."""
    orig = cls._dummy_run
    if _already(orig):
        return

    def _dummy_run(self, *args, **kwargs):
        global _v1_dummy_depth
        _v1_dummy_depth += 1
        try:
            return orig(self, *args, **kwargs)
        finally:
            _v1_dummy_depth -= 1

    cls._dummy_run = _tag(_dummy_run)


def install() -> None:
    """Hook vLLM's block tables so the metadata builder can read them on the host (idempotent)."""
    try:
        from vllm.v1.worker.block_table import BlockTable
        from vllm.v1.worker.gpu_model_runner import GPUModelRunner

        _remember_instances(BlockTable, _v1_tables)
        install_v1_dummy(GPUModelRunner)
    except ImportError:
        pass
    try:
        from vllm.v1.worker.gpu.block_table import BlockTables

        install_v2(BlockTables)
    except ImportError:
        pass


def _v1_owner(ptr: int):
    for t in list(_v1_tables):
        buf = getattr(t, "block_table", None)
        if buf is not None and buf.gpu.data_ptr() == ptr:
            return t
    return None


def _v2_owner(ptr: int):
    for t in list(_v2_tables):
        for g, inp in enumerate(t.input_block_tables):
            if inp.data_ptr() == ptr:
                return t, g
    return None


def is_dummy_step(cm) -> bool:
    """Whether ``cm`` belongs to one of vLLM's dummy steps (all-PAD slot mapping)."""
    ptr = cm.block_table_tensor.data_ptr()
    if _v1_owner(ptr) is not None:
        return _v1_dummy_depth > 0
    hit = _v2_owner(ptr)
    return bool(hit and getattr(hit[0], "_echokv_dummy", False))


def _host_table(cm, block_size: int):
    """(host block table, batch row -> table row map or None) for ``cm``, or None if untrusted."""
    ptr = cm.block_table_tensor.data_ptr()
    t = _v1_owner(ptr)
    if t is not None:
        if t.block_size != block_size or t.dcp_world_size != 1 or t.pcp_world_size != 1 or _v1_dummy_depth:
            return None
        return t.block_table.np, None
    hit = _v2_owner(ptr)
    if hit is not None:
        t, g = hit
        req_idx = getattr(cm, "req_idx", None)
        if t.block_sizes[g] != block_size or t.cp_size != 1 or req_idx is None or getattr(t, "_echokv_dummy", False):
            return None
        return t._echokv_np[g], np.asarray(req_idx, dtype=np.int64)
    return None


def host_lens_and_slots(cm, block_size: int):
    """``(seq_lens[:num_reqs], slot_mapping[:num_actual_tokens])`` as CPU tensors, or None.

    None when the host copies cannot be trusted (a dummy step, no CPU sequence lengths, an unknown
    block table, context parallelism); the caller then copies the device tensors back.  Padding
    tokens map to -1, as on the device.
    """
    seq = getattr(cm, "seq_lens_cpu_upper_bound", None)
    if seq is None:
        return None
    found = _host_table(cm, block_size)
    if found is None:
        return None
    table, row_map = found
    n = cm.num_reqs
    starts = cm.query_start_loc_cpu[: n + 1].numpy().astype(np.int64)
    lens = seq[:n].numpy().astype(np.int64)
    qlen = np.diff(starts)
    total = int(starts[-1])
    if total > cm.num_actual_tokens:
        return None
    req = np.repeat(np.arange(n), qlen)
    pos = np.arange(total) - starts[:-1][req] + (lens - qlen)[req]
    if row_map is not None and req.size and req[-1] >= row_map.size:
        return None
    rows = req if row_map is None else row_map[req]
    slots = np.full(cm.num_actual_tokens, -1, dtype=np.int64)
    slots[:total] = table[rows, pos // block_size].astype(np.int64) * block_size + pos % block_size
    return torch.from_numpy(lens), torch.from_numpy(slots)
