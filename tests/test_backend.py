"""The vLLM adapter driven the way vLLM's model runner drives it (builder.build once per step, then
do_kv_cache_update and forward per layer), with stand-ins for vLLM's config, layers and forward
context, against the numpy oracle: page bytes bit-exact, attention within the bf16 tolerance."""

from types import SimpleNamespace

import numpy as np
import pytest

from oracle import echokv_oracle as O

H, HQ, D, BS, BLOCKS, LAYERS = 2, 8, 128, 16, 40, 2
ENV = {"ECHOKV_MEM_BITS": "8", "ECHOKV_K_GROUP": "16", "ECHOKV_CANARY_INTERVAL": "2", "ECHOKV_KREF_WINDOW": "32",
       "ECHOKV_RESIDUAL_SLOTS": "8", "ECHOKV_CANARY_MAX_Q": "4"}


@pytest.fixture
def env(monkeypatch):
    for k, v in ENV.items():
        monkeypatch.setenv(k, v)
    for k in ("ECHOKV_FIXED_BITS", "ECHOKV_INIT_BITS", "ECHOKV_V_GROUP", "ECHOKV_CUDAGRAPH"):
        monkeypatch.delenv(k, raising=False)


def test_backend_contract(env, monkeypatch):
    import torch
    from echokv_b200 import backend as B

    be = B.EchoKVAttentionBackend
    assert be.get_name() == "CUSTOM" and be.forward_includes_kv_cache_update is False
    assert be.get_impl_cls() is B.EchoKVAttentionImpl and be.get_builder_cls() is B.EchoKVMetadataBuilder
    assert be.supports_block_size(None) and be.supports_block_size(32) and not be.supports_block_size(24)
    assert be.supports_head_size(128) and not be.supports_head_size(80)
    assert be.supports_attn_type("decoder") and not be.supports_attn_type("encoder")
    assert be.supported_dtypes == [torch.float16, torch.bfloat16, torch.float32]
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class Spec:
        num_kv_heads: int = 8
        head_size: int = 128
        head_size_v: int = 128
        num_head_slots: int = 2
        state_content_bytes: int = 0

    got = be.customize_spec(Spec())
    assert got.num_head_slots == 1 and got.state_content_bytes == 2436  # H 8, D 128, mem 8, K group 16
    with pytest.raises(NotImplementedError):
        be.customize_spec(Spec(head_size_v=64))
    for bad in ({"alibi_slopes": [1.0]}, {"sliding_window": 128}, {"logits_soft_cap": 30.0}, {"sinks": torch.zeros(2)},
                {"kv_sharing_target_layer_name": "x"}, {"attn_type": "encoder"}):
        with pytest.raises(NotImplementedError, match="EchoKV does not support"):
            B.EchoKVAttentionImpl(HQ, D, 0.1, H, **bad)
    impl = B.EchoKVAttentionImpl(HQ, D, 0.1, H)
    assert impl.residual.shape == (9, 16, H, D) and impl.kref_buf.shape == (32, H, D) and impl.stash.shape == (4, HQ, D)
    with pytest.raises(NotImplementedError, match="output quantization"):
        impl.forward(None, None, None, None, None, None, None, output_scale=torch.ones(1))
    support = B.EchoKVMetadataBuilder.get_cudagraph_support(None, None)
    assert support == B.AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
    monkeypatch.setenv("ECHOKV_CUDAGRAPH", "0")
    assert B.EchoKVMetadataBuilder.get_cudagraph_support(None, None) == B.AttentionCGSupport.NEVER


def test_split_batch_and_canary_schedule():
    from echokv_b200.backend import CanarySchedule, split_batch

    # decode-only with a padding request: one entry per request, padding has length 0
    rows, reqs, lens, prefill, p_reqs, last, ctx = split_batch(np.array([0, 1, 2, 2]), np.array([9, 30, 0]), 4)
    assert rows.tolist() == [0, 1, 2] and reqs.tolist() == [0, 1, 2] and lens.tolist() == [9, 30, 0]
    assert not prefill and last.tolist() == [0, 1] and ctx.tolist() == [9, 30]
    # mixed: request 1 is a 5-token chunk ending at 12, request 2 is idle
    rows, reqs, lens, prefill, p_reqs, last, ctx = split_batch(np.array([0, 1, 6, 6, 7]), np.array([4, 12, 0, 8]), 7)
    assert rows.tolist() == [0, 6] and reqs.tolist() == [0, 3] and lens.tolist() == [4, 8]
    assert prefill == [(1, 6, 12, 0)] and p_reqs == [1] and last.tolist() == [0, 5, 6]
    sched = CanarySchedule(interval=3, max_q=2)
    fires = [sched.rows_for(False, np.array([4, 7, 9]), np.array([10, 20, 30]))[1] for _ in range(6)]
    assert fires == [False, False, True, False, False, True] and sched.stashed == (2, 15.0)
    sched = CanarySchedule(interval=1, max_q=2)
    assert sched.rows_for(True, np.array([1]), np.array([5]))[1] is False and sched.steps == 0  # dummy steps do not count
    assert sched.rows_for(False, np.array([], dtype=np.int64), np.array([]))[1] is False and sched.armed  # waits for a live row
    rows, fire = sched.rows_for(False, np.array([3]), np.array([8]))
    assert fire and rows.tolist() == [3, 0]


class Harness:
    """Plays vLLM: owns block tables, builds common metadata, calls the builder and the impls."""

    def __init__(self, monkeypatch, dtype):
        import torch
        from vllm.model_executor.layers.attention_layer_base import AttentionLayerBase

        from echokv_b200 import backend as B

        self.torch, self.B, self.dtype = torch, B, dtype
        monkeypatch.setattr(B, "_model_dtype", lambda: dtype)
        self.ctx = SimpleNamespace(attn_metadata=None)
        monkeypatch.setattr(B, "get_forward_context", lambda: self.ctx)

        class Layer(torch.nn.Module, AttentionLayerBase):
            def __init__(self, name, impl):
                super().__init__()
                self.layer_name, self.impl, self.kv_cache = name, impl, None

            def get_attn_backend(self):
                return B.EchoKVAttentionBackend

            def get_kv_cache_spec(self, vllm_config):
                return None

        self.scale = D ** -0.5
        self.layers = [Layer(f"model.layers.{i}.self_attn.attn", B.EchoKVAttentionImpl(HQ, D, self.scale, H))
                       for i in range(LAYERS)]
        self.tiers = [8, 4]
        for layer, bits in zip(self.layers, self.tiers):
            layer.impl.controller.bits = bits
        names = [layer.layer_name for layer in self.layers]
        self.vllm_config = SimpleNamespace(
            speculative_config=None, parallel_config=None, scheduler_config=SimpleNamespace(max_num_seqs=8),
            compilation_config=SimpleNamespace(max_cudagraph_capture_size=16,
                                               static_forward_context=dict(zip(names, self.layers))),
            model_config=SimpleNamespace(max_model_len=512, dtype=dtype, get_num_attention_heads=lambda pc: HQ))
        spec = SimpleNamespace(block_size=BS, num_kv_heads=H, head_size=D)
        self.builder = B.EchoKVMetadataBuilder(spec, names, self.vllm_config, torch.device("cuda"))
        self.per_token = B.TieredLayout.per_token_bytes(H, D, 8, 16, 32)
        self.table = np.zeros((4, 16), dtype=np.int32)
        self.table[:3, :12] = np.random.default_rng(1).permutation(np.arange(1, BLOCKS))[:36].reshape(3, 12)
        self.lens = [0, 0, 0, 0]
        self.rng = np.random.default_rng(2)
        lay = O.Layout(H, D, BS, 8, 16, 32)
        self.oracles = [O.Store(lay, BLOCKS, page_bytes=BS * self.per_token, residual_slots=8, residual_dtype="bf16",
                                kref_window=32) for _ in range(LAYERS)]
        self.krefs = [np.zeros((32, H, D), dtype=np.float32) for _ in range(LAYERS)]

    def allocate_caches(self):
        for layer in self.layers:
            layer.kv_cache = self.torch.zeros(BLOCKS, 1, BS, self.per_token, dtype=self.torch.uint8, device="cuda")

    def step(self, new_tokens, pad_to=None):
        """One engine step: request r appends new_tokens[r] tokens.  Returns per-layer (got, want, rows)."""
        torch = self.torch
        starts, slots = [0], []
        for r, n in enumerate(new_tokens):
            for p in range(self.lens[r], self.lens[r] + n):
                slots.append(int(self.table[r, p // BS]) * BS + p % BS)
            self.lens[r] += n
            starts.append(starts[-1] + n)
        t = starts[-1]
        padded = pad_to or t
        lens = [self.lens[r] if n else 0 for r, n in enumerate(new_tokens)]
        cm = SimpleNamespace(
            causal=True, num_reqs=len(new_tokens), num_actual_tokens=padded,
            query_start_loc_cpu=torch.tensor(starts, dtype=torch.int32), seq_lens=torch.tensor(lens, dtype=torch.int32).cuda(),
            seq_lens_cpu_upper_bound=torch.tensor(lens, dtype=torch.int32),
            slot_mapping=torch.tensor(slots + [-1] * (padded - t), dtype=torch.int64).cuda(),
            block_table_tensor=torch.from_numpy(self.table).cuda())
        md = self.builder.build(0, cm)
        self.ctx.attn_metadata = {layer.layer_name: md for layer in self.layers}
        results = []
        slots_np = np.array(slots + [-1] * (padded - t), dtype=np.int64)
        for li, layer in enumerate(self.layers):
            q, k, v = (torch.from_numpy(self.rng.standard_normal((padded, n, D), dtype=np.float32)).to(self.dtype)
                       for n in (HQ, H, H))
            out = torch.zeros(padded, HQ * D, dtype=self.dtype, device="cuda")
            qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
            layer.impl.do_kv_cache_update(layer, kd, vd, layer.kv_cache, cm.slot_mapping)
            layer.impl.forward(layer, qd, kd, vd, layer.kv_cache, md, out)
            st = self.oracles[li]
            st.write(k.float().numpy(), v.float().numpy(), slots_np, layer.impl.controller.bits, kref=self.krefs[li])
            want = np.zeros((padded, HQ, D), dtype=np.float32)
            live = []
            for r, n in enumerate(new_tokens):
                if n == 0:
                    continue
                qs, qe = starts[r], starts[r + 1]
                live.extend(range(qs, qe))
                if n == 1:
                    want[qs] = O.decode_attention(st, q[qs:qe].float().numpy(), self.table[r:r + 1], [self.lens[r]], self.scale)[0]
                else:
                    rnd = (lambda a: torch.from_numpy(a).to(self.dtype).float().numpy())
                    want[qs:qe] = O.prefill_attention(st, q.float().numpy(), [(qs, qe, self.lens[r], 0)], [r], self.table,
                                                      self.scale, round_kv=rnd)[qs:qe]
            results.append((out.view(padded, HQ, D).float().cpu().numpy(), want, live))
        return md, results


@pytest.mark.gpu
def test_engine_steps_match_the_oracle(env, monkeypatch):
    import torch

    hs = Harness(monkeypatch, torch.bfloat16)
    # memory profiling: no KV cache yet -> metadata without a write plan, forward leaves the output alone
    md, res = None, None
    cm_tokens = [3, 0, 0, 0]
    saved = list(hs.lens)
    md = hs.builder.build(0, SimpleNamespace(
        causal=True, num_reqs=1, num_actual_tokens=3, query_start_loc_cpu=torch.tensor([0, 3], dtype=torch.int32),
        seq_lens=torch.tensor([3], dtype=torch.int32).cuda(), seq_lens_cpu_upper_bound=torch.tensor([3], dtype=torch.int32),
        slot_mapping=torch.full((3,), -1, dtype=torch.int64).cuda(), block_table_tensor=torch.from_numpy(hs.table).cuda()))
    assert md.write is None and hs.builder.runner is None
    out = torch.ones(3, HQ * D, device="cuda")
    impl0 = hs.layers[0].impl
    assert impl0.forward(hs.layers[0], out, out, out, None, md, out) is out and impl0.forward_calls == 0
    hs.lens = saved
    hs.allocate_caches()

    plan = [
        ([40, 70, 0, 0], None),      # two prefill chunks (row path 40, dense path 70)
        ([1, 1, 150, 0], None),      # mixed: two decodes and a long prefill (dense path)
        ([1, 1, 1, 0], None),        # decode-only
        ([1, 1, 1, 0], 8),           # decode-only, padded like a captured graph size
        ([30, 1, 1, 0], None),       # a second chunk for request 0 (ctx 73 after it)
        ([1, 1, 1, 0], None),
    ]
    for new_tokens, pad in plan:
        md, res = hs.step(new_tokens, pad)
        assert md.write is not None and md.num_splits == hs.builder.num_splits
        for li, (got, want, live) in enumerate(res):
            err = np.abs(got[live] - want[live]).max()
            assert err <= 3e-2, (new_tokens, li, err)
            rest = np.setdiff1d(np.arange(got.shape[0]), live)
            assert not got[rest].any()  # padding rows stay untouched
    for li, layer in enumerate(hs.layers):
        st = hs.oracles[li]
        got = layer.kv_cache.view(-1).cpu().numpy()
        assert np.array_equal(got, st.backing[: got.size]), f"layer {li} pages differ"
        assert layer.impl.store.tokens_written[hs.tiers[li]] > 0 and layer.impl.forward_calls == len(plan)
        np.testing.assert_array_equal(layer.impl.kref_buf.cpu().numpy(), hs.krefs[li])
    # canary: interval 2 -> fires on steps 2, 4, 6; each is measured at the following build
    c = hs.builder.canary
    assert c.steps == len(plan) and c.stashed is not None and c.unread is not None
    deltas, ctx = c.unread
    assert deltas.shape == (LAYERS, 3) and torch.isfinite(deltas).all() and ctx > 0
    assert all(layer.impl.controller.fires >= 1 for layer in hs.layers)
    # the control surface sees the same layers
    from echokv_b200 import control

    model = torch.nn.Module()
    model.layers = torch.nn.ModuleList(hs.layers)
    state = control.get_state(model)
    assert state["tier_vector"] == control.get_tier_vector(model) == [layer.impl.controller.bits for layer in hs.layers]
    assert state["layers"][0]["forward_calls"] == len(plan) and state["avg_stored_bits"] is not None
    assert control.set_frozen(model, True) == LAYERS and hs.layers[0].impl.controller.params.frozen
    assert control.set_tier_vector(model, 2) == LAYERS and control.get_tier_vector(model) == [2, 2]
    with pytest.raises(ValueError):
        control.set_tier_vector(model, [8])
    assert control.reset_counters(model) == LAYERS and hs.layers[0].impl.forward_calls == 0
