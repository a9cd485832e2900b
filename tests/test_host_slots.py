"""Host slot mapping against vLLM's per-token rule, with stand-ins for both runners' block tables
(the reference's tests/echokv_vllm/test_host_slots.py covers the same cases)."""

from types import SimpleNamespace

import numpy as np
import torch

from echokv_b200 import host_slots as HS

BLOCK = 16


def device_rule(rows, starts, lens, num_tokens):
    """slot = table[request, pos // BLOCK] * BLOCK + pos % BLOCK for the last (query length) positions."""
    out = np.full(num_tokens, -1, dtype=np.int64)
    for r, n in enumerate(lens):
        q = starts[r + 1] - starts[r]
        for i in range(q):
            pos = n - q + i
            out[starts[r] + i] = rows[r][pos // BLOCK] * BLOCK + pos % BLOCK
    return torch.from_numpy(out)


def batch(table, starts, lens, num_tokens, req_idx=None):
    return SimpleNamespace(seq_lens_cpu_upper_bound=torch.tensor(lens, dtype=torch.int32), block_table_tensor=table,
                           num_reqs=len(lens), query_start_loc_cpu=torch.tensor(starts, dtype=torch.int32),
                           num_actual_tokens=num_tokens, req_idx=req_idx)


class SlotTables:
    """What the hooks use of the V2 runner's block tables: per-slot GPU tables written through
    ``append_block_ids``, a staging table the batch reads, and the two slot-mapping entry points."""

    def __init__(self, slots: int, width: int) -> None:
        self.num_kv_cache_groups, self.block_sizes, self.cp_size = 1, [BLOCK], 1
        self.block_tables = [SimpleNamespace(gpu=torch.zeros(slots, width, dtype=torch.int32))]
        self.num_blocks = SimpleNamespace(np=np.zeros((1, slots), dtype=np.int32))
        self.input_block_tables = [torch.zeros(slots, width, dtype=torch.int32)]

    def append_block_ids(self, req_index, new_block_ids, overwrite):
        at = 0 if overwrite else int(self.num_blocks.np[0, req_index])
        for k, b in enumerate(new_block_ids[0]):
            self.block_tables[0].gpu[req_index, at + k] = b
        self.num_blocks.np[0, req_index] = at + len(new_block_ids[0])

    def compute_slot_mappings(self):
        return None

    def get_dummy_slot_mappings(self, n):
        return None

    def stage(self, slots):
        self.input_block_tables[0][: len(slots)] = self.block_tables[0].gpu[torch.as_tensor(slots)]
        return self.input_block_tables[0][: len(slots)]


def test_v2_mirror_follows_growth_and_slot_reuse():
    HS.install_v2(SlotTables)
    HS.install_v2(SlotTables)  # idempotent
    t = SlotTables(4, 8)
    t.append_block_ids(3, ([12, 5],), True)
    t.append_block_ids(1, ([8],), True)
    t.append_block_ids(3, ([2],), False)      # the request in slot 3 grows
    t.append_block_ids(1, ([6, 14],), True)   # slot 1 handed to a new request
    # row 0: slot 3 decoding at position 33; row 1: slot 1 prefilling 18 tokens; row 2: padding
    starts, lens, n = [0, 1, 19, 19], [34, 18, 0], 22
    cm = batch(t.stage([3, 1]), starts, lens, n, np.array([3, 1]))
    got_lens, got = HS.host_lens_and_slots(cm, BLOCK)
    assert got_lens.tolist() == lens
    assert torch.equal(got, device_rule([[12, 5, 2], [6, 14], []], starts, lens, n))
    assert (got[19:] == -1).all()


def test_chunked_prefill_positions_start_after_the_computed_prefix():
    HS.install_v2(SlotTables)
    t = SlotTables(2, 8)
    t.append_block_ids(0, ([3, 9, 4],), True)
    starts, lens = [0, 10], [37]  # 27 tokens already in the cache, 10 new
    got = HS.host_lens_and_slots(batch(t.stage([0]), starts, lens, 10, np.array([0])), BLOCK)[1]
    assert torch.equal(got, device_rule([[3, 9, 4]], starts, lens, 10))


def test_untrusted_inputs_return_none():
    HS.install_v2(SlotTables)
    t = SlotTables(2, 4)
    t.append_block_ids(0, ([1],), True)
    cm = batch(t.stage([0]), [0, 1], [3], 1, np.array([0]))
    assert HS.host_lens_and_slots(cm, BLOCK) is not None
    assert HS.host_lens_and_slots(cm, 2 * BLOCK) is None                                 # other block size
    assert HS.host_lens_and_slots(batch(torch.zeros(1, 4), [0, 1], [3], 1), BLOCK) is None  # unknown table
    cm.req_idx = None
    assert HS.host_lens_and_slots(cm, BLOCK) is None                                     # no slot map
    cm.req_idx, cm.seq_lens_cpu_upper_bound = np.array([0]), None
    assert HS.host_lens_and_slots(cm, BLOCK) is None                                     # no CPU lengths


def test_v1_table_is_read_by_batch_row():
    class RowTable:
        def __init__(self):
            self.block_size, self.dcp_world_size, self.pcp_world_size = BLOCK, 1, 1
            rows = np.array([[4, 6, 0, 0], [2, 0, 0, 0], [0, 0, 0, 0]], dtype=np.int32)
            self.block_table = SimpleNamespace(gpu=torch.from_numpy(rows.copy()), np=rows)

    HS._remember_instances(RowTable, HS._v1_tables)
    t = RowTable()
    starts, lens = [0, 3, 4], [20, 9]
    cm = batch(t.block_table.gpu, starts, lens, 4)
    assert not HS.is_dummy_step(cm)
    assert torch.equal(HS.host_lens_and_slots(cm, BLOCK)[1], device_rule(t.block_table.np, starts, lens, 4))

    class Runner:
        def _dummy_run(self, probe):
            return probe()

    HS.install_v1_dummy(Runner)
    inside = Runner()._dummy_run(lambda: (HS.is_dummy_step(cm), HS.host_lens_and_slots(cm, BLOCK)))
    assert inside == (True, None) and HS._v1_dummy_depth == 0


def test_v2_dummy_steps_take_the_device_copy():
    HS.install_v2(SlotTables)
    t = SlotTables(2, 4)
    t.append_block_ids(0, ([3],), True)
    cm = batch(t.stage([0]), [0, 1], [5], 1, np.array([0]))
    t.compute_slot_mappings()
    assert HS.host_lens_and_slots(cm, BLOCK) is not None and not HS.is_dummy_step(cm)
    t.get_dummy_slot_mappings(1)  # warmup, graph capture, an idle data-parallel rank
    assert HS.host_lens_and_slots(cm, BLOCK) is None and HS.is_dummy_step(cm)
    t.compute_slot_mappings()
    assert HS.host_lens_and_slots(cm, BLOCK) is not None


def test_null_block_redirect_is_mirrored():
    HS.install_v2(SlotTables)
    t = SlotTables(1, 4)
    t.redirect_writes_to_null_block = True
    t.append_block_ids(0, ([7, 8],), True)
    assert t._echokv_np[0][0, :2].tolist() == [0, 0]


def test_plugin_entry_point_is_declared(tmp_path, monkeypatch):
    """pyproject.toml declares `echokv = echokv_b200.plugin:register` in the `vllm.general_plugins` group
    (pyproject.toml:12-13 of the reference): build the package metadata and find it the way vLLM does."""
    import importlib.metadata as md
    import os
    from pathlib import Path

    import setuptools.build_meta as backend

    root = Path(__file__).resolve().parent.parent
    monkeypatch.chdir(root)
    before = set(os.listdir(root))
    try:
        info = backend.prepare_metadata_for_build_wheel(str(tmp_path))
    finally:
        import shutil
        for name in set(os.listdir(root)) - before:  # setuptools leaves an egg-info folder beside the sources
            shutil.rmtree(root / name, ignore_errors=True)
    dist = md.PathDistribution(tmp_path / info)
    assert dist.metadata["Name"] == "echokv-b200"
    eps = [e for e in dist.entry_points if e.group == "vllm.general_plugins"]
    assert [(e.name, e.value) for e in eps] == [("echokv", "echokv_b200.plugin:register")]
    register = eps[0].load()
    monkeypatch.delenv("ECHOKV_ENABLE", raising=False)
    register()  # without ECHOKV_ENABLE=1 the call touches nothing (plugin.py:17-28 of the reference)


def test_page_size_shim_for_vllm_without_customize_spec(monkeypatch):
    """On vLLM releases that lack ``AttentionBackend.customize_spec`` the plugin makes the attention layers it serves
    declare their page through ``TQFullAttentionSpec``: page bytes = block_size * bytes per token of the tiered store
    (rounded up to whole slots per head), and the backend's cache shape covers exactly that page."""
    import types

    import pytest
    import torch

    vllm = pytest.importorskip("vllm")  # noqa: F841
    from echokv_b200 import vllm_compat
    from echokv_b200.tiered_cache import TieredLayout

    if not vllm_compat.needs_spec_patch():
        pytest.skip("this vLLM has customize_spec; the shim is not used")
    monkeypatch.setenv("ECHOKV_MEM_BITS", "4")
    monkeypatch.setenv("ECHOKV_K_GROUP", "32")
    from vllm.model_executor.layers.attention.attention import Attention
    from vllm.v1.attention.backend import AttentionType
    from vllm.v1.kv_cache_interface import FullAttentionSpec, TQFullAttentionSpec

    from echokv_b200.backend import EchoKVAttentionBackend

    assert vllm_compat.install()
    cfg = types.SimpleNamespace(cache_config=types.SimpleNamespace(block_size=64),
                                model_config=types.SimpleNamespace(use_mla=False))

    def layer(backend):
        return types.SimpleNamespace(attn_type=AttentionType.DECODER, kv_cache_dtype="auto", sliding_window=None, num_kv_heads=8,
                                     head_size=128, head_size_v=128, kv_cache_torch_dtype=torch.bfloat16,
                                     get_attn_backend=lambda: backend)

    ours = Attention.get_kv_cache_spec(layer(EchoKVAttentionBackend), cfg)
    assert isinstance(ours, TQFullAttentionSpec)
    per_token = TieredLayout.per_token_bytes(8, 128, 4, 32, 32)
    assert per_token == 1284 and vllm_compat.slot_bytes(8, 128) == 164
    assert ours.page_size_bytes == 64 * 8 * 164 >= 64 * per_token
    stock = FullAttentionSpec(block_size=64, num_kv_heads=8, head_size=128, dtype=torch.bfloat16)
    assert stock.page_size_bytes / ours.page_size_bytes > 3.0  # the capacity the reference advertises for INT4
    shape = EchoKVAttentionBackend.get_kv_cache_shape(10, 64, 8, 128)
    assert shape[0] == 10 and shape[1] == 1 and shape[2] == 64
    other = Attention.get_kv_cache_spec(layer(type("Other", (), {"__module__": "vllm.somewhere"})), cfg)
    assert type(other) is FullAttentionSpec
