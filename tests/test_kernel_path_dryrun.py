"""Dry run of the kernel route on CPU: every entry point of the kernel library is replaced by a recorder that
launches nothing, so one training step of a tiny bf16 model walks the same Python code a GPU step does (autograd
functions, push targets, kept dispatch, fp8 recipes, dead outputs of the recomputed block) and fails on any
host-side mistake (wrong argument lists, wrong number of returned gradients, shape bookkeeping).  Numbers are
meaningless here; the GPU suite checks those."""
import pytest
import torch


@pytest.fixture
def dry(monkeypatch):
    from system_lab_b200 import ops
    from system_lab_b200.ops import cuda as cops
    try:
        cops.lib()
    except Exception as e:
        pytest.skip(f"kernel library not built: {e}")
    class Calls(list):
        waited_in_kernel = 0

    calls = Calls()

    def fake_call(name, *args):
        assert name in cops._SIGS, f"unregistered entry point {name}"
        assert len(args) == len(cops._SIGS[name]), (name, len(args), len(cops._SIGS[name]))
        for a, kind in zip(args, cops._SIGS[name]):
            if kind == "p":
                assert a is None or isinstance(a, (torch.Tensor, int)), (name, type(a))
            elif kind in "il":
                assert isinstance(a, int) and not isinstance(a, bool), (name, kind, type(a), a)
            elif kind == "f":
                assert isinstance(a, (int, float)), (name, type(a))
        for a in args:                    # index-like buffers must hold valid indices for the host-side torch ops
            if isinstance(a, torch.Tensor) and a.dtype in (torch.int32, torch.int64):
                a.data.zero_()
        calls.append(name)
        if name == "slab_grouped_gemm_bf16" and args[13] is not None:
            calls.waited_in_kernel += 1               # the GEMM took per-expert arrival flags
        cops.LAUNCHES[0] += 1
        return 0

    monkeypatch.setattr(cops, "call", fake_call)
    monkeypatch.setattr(cops, "stream", lambda: 0)
    monkeypatch.setattr(ops, "use_kernels", lambda *t: True)
    monkeypatch.setattr(ops, "set_kernel_mode", lambda mode: None)
    return calls


def _trainer(extra, dispatcher_kw=None):
    from system_lab_b200.config import Config
    from system_lab_b200.moe.fused_dispatch import FusedDispatcher
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "params_dtype=bf16", "global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=1",
        "hidden_size=256", "moe_ffn_hidden_size=128", "kv_channels=64", "device=cpu", "moe_pad_expert_rows_to=128"] + extra)
    tr = Trainer(cfg)
    m = cfg.model
    d = FusedDispatcher(tr.mesh, m.num_experts, m.moe_router_topk, m.hidden_size,
                        cfg.train.micro_batch_size * m.seq_length, 128, torch.device("cpu"),
                        clone_outputs=not (tr.engine.recompute or tr.engine.selective), **(dispatcher_kw or {}))
    for f in tr.engine.moe_ffns():
        f.dispatcher = d
    tr.engine.dispatcher = d
    return tr, d


@pytest.mark.parametrize("extra,kw", [
    (["recompute_granularity=selective"], {}),
    (["recompute_granularity=selective"], {"push": True}),
    (["recompute_granularity=selective", "moe_keep_dispatched_factor=-1"], {"push": True, "keep_factor": -1.0}),
    (["recompute_granularity=selective", "moe_keep_dispatched_factor=2"], {"keep_factor": 2.0}),
    (["recompute_granularity=selective", "moe_keep_dispatched_factor=-1"], {"keep_factor": -1.0}),   # kept rows < capacity, pull combine
    (["recompute_granularity=selective", "moe_keep_dispatched_factor=0.25"], {"keep_factor": 0.25}),
    (["recompute_granularity=full"], {"push": True}),
    (["recompute_granularity=none"], {"push": True}),
    (["recompute_granularity=selective", "fp8=true", "fp8_recipe=rowwise"], {"push": True}),
    (["recompute_granularity=selective", "fp8=true", "fp8_recipe=blockwise"], {}),
    (["recompute_granularity=selective", "fp8=true", "fp8_recipe=tensorwise"], {"push": True}),
    (["recompute_granularity=selective", "optimizer_in_backward=true", "master_weights=false",
      "optimizer_state_dtype=fp8", "global_batch_size=2"], {}),
    (["recompute_granularity=selective", "global_batch_size=8"], {"push": True}),          # four micro-batches
])
def test_one_step_walks_the_kernel_route(dry, extra, kw):
    tr, d = _trainer(extra, kw)
    out = tr.train_step()
    assert out["loss"].shape == ()
    names = set(dry)
    assert {"slab_grouped_gemm_bf16", "slab_moe_plan_slots", "slab_adamw"} <= names
    assert "slab_moe_scatter_sorted" in names            # rows travel expert by expert, one flag per (source, expert)
    if kw.get("push"):
        assert "slab_grouped_gemm_bf16_push" in names and "slab_moe_reduce_pairs" in names
        assert d._pending_push == {}                        # every push was consumed by its reduction
        assert d.push_epoch == dry.count("slab_grouped_gemm_bf16_push") == dry.count("slab_moe_reduce_pairs")
    if "fp8=true" in extra:
        assert ("slab_grouped_gemm_fp8_rowwise" in names) or ("slab_grouped_gemm_fp8" in names)
    gbs = next((int(x.split("=")[1]) for x in extra if x.startswith("global_batch_size=")), 4)
    layers, nmb = 2, gbs // 2                                   # micro-batches of 2 sequences on one rank
    scatters = dry.count("slab_moe_scatter") + dry.count("slab_moe_scatter_sorted")
    # every expert-ordered scatter is honoured exactly once: by a GEMM that waits inside the kernel or by a wait kernel
    assert dry.count("slab_moe_scatter_sorted") == dry.waited_in_kernel + dry.count("slab_moe_wait_experts")
    if "fp8=true" not in extra and not any(x.startswith("moe_keep_dispatched_factor=") for x in extra) \
            and "recompute_granularity=none" not in extra:        # kept activations are copies: those wait first
        assert dry.count("slab_moe_wait_experts") == 0          # bf16 route: no wait for a whole exchange anywhere
    if any(x.startswith("moe_keep_dispatched_factor=") for x in extra):
        assert scatters == layers * nmb * 2                  # forward dispatch + backward of combine; no re-dispatch
    elif "recompute_granularity=none" in extra:
        assert scatters == layers * nmb * 2
    else:
        assert scatters == layers * nmb * 3                  # + the recomputed block's dispatch


MLA = ["attention_type=mla", "q_lora_rank=64", "kv_lora_rank=64", "qk_nope_head_dim=32", "qk_rope_head_dim=32",
       "v_head_dim=32", "moe_shared_expert_intermediate_size=128", "moe_router_score_function=sigmoid",
       "moe_router_load_balancing_type=bias", "first_k_dense=1", "ffn_hidden_size=256", "num_layers=3"]


@pytest.mark.parametrize("extra,kw", [
    (MLA + ["recompute_granularity=selective"], {"push": True}),
    (["sliding_window=16", "recompute_granularity=full", "num_layers=2"], {}),
    (["moe_aux_loss_coeff=0.01", "recompute_granularity=selective"], {"push": True}),      # aux loss carried through the recompute node
    (["moe_router_force_load_balancing=true", "recompute_granularity=selective"], {}),
    (["moe_expert_relocation_interval=1", "moe_expert_relocation_min_gain=0.0", "recompute_granularity=selective"], {}),
    (MLA + ["recompute_granularity=selective", "moe_keep_dispatched_factor=-1"], {"push": True, "keep_factor": -1.0}),
    (["recompute_granularity=selective", "moe_keep_dispatched_factor=-1", "fp8=true", "global_batch_size=8"],
     {"keep_factor": -1.0}),
    (["recompute_granularity=selective", "optimizer_in_backward=true", "global_batch_size=2",
      "moe_keep_dispatched_factor=-1"], {"push": True, "keep_factor": -1.0}),
    (["recompute_granularity=full", "fp8=true", "fp8_recipe=blockwise", "num_layers_at_start_in_bf16=1"], {"push": True}),
])
def test_model_variants_walk_the_kernel_route(dry, extra, kw):
    tr, d = _trainer(extra, kw)
    for _ in range(2):
        out = tr.train_step()
        assert out["loss"].shape == ()
    assert "slab_grouped_gemm_bf16" in set(dry) and d._pending_push == {}
    tr.evaluate(1)


def test_attention_kernel_binding_argument_list(dry, monkeypatch):
    """The opt-in attention forward: strides of packed qkv slices, argument list against the registered signature,
    and the autograd wrapper's library backward."""
    from system_lab_b200.ops import attention_kernel as ak, cuda as cops
    monkeypatch.setattr(cops, "status_word", lambda dev: torch.zeros(1, dtype=torch.int32))
    b, s, hq, hkv, d = 2, 256, 4, 2, 64
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d, dtype=torch.bfloat16)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    assert ak._row_stride(q) == ak._row_stride(k) == ak._row_stride(v) == (hq + 2 * hkv) * d
    assert ak._row_stride(q.transpose(1, 2)) is None                  # heads not contiguous: refused
    assert not ak.shape_ok(q, k, v, 0)                                 # CPU tensors never take the kernel
    out, lse = ak.forward(q, k, v, 0.125, 128)
    assert out.shape == (b, s, hq, d) and lse.shape == (b, hq, s) and dry[-1] == "slab_attn_fwd"
    q2 = q.detach().float().requires_grad_(True)
    o = ak.attention(q2, k.float(), v.float(), 0.125, 0)              # backward goes through the library attention
    o.sum().backward()
    assert q2.grad is not None and q2.grad.shape == q2.shape


def test_hidden_with_half_a_row_tile_takes_the_kernel_route_when_opted_in(dry, monkeypatch):
    """hidden % 128 == 64 (the GPT-OSS width 2880 = 22.5 x 128): with the opt-in switch the expert GEMMs stay on the
    kernel route (wgrad writes its last row tile with guarded stores) and the bf16 scatter takes any H % 8 == 0."""
    from system_lab_b200.ops import cuda as cops
    monkeypatch.setattr(cops, "_N_MULTIPLE", 64)
    tr, d = _trainer(["recompute_granularity=selective", "hidden_size=320", "moe_ffn_hidden_size=192"], {"push": True})
    tr.train_step()
    assert dry.count("slab_grouped_gemm_bf16") + dry.count("slab_grouped_gemm_bf16_push") >= 7 * len(tr.engine.moe_ffns())


def test_lora_dense_model_on_the_kernel_route(dry):
    """A dense bf16 model with LoRA adapters: the fused cross entropy skips the frozen head's weight gradient and the
    optimizer only sees the adapter groups."""
    from system_lab_b200.config import Config
    from system_lab_b200.trainer.loop import Trainer
    cfg = Config.load(preset="simplemoe-tiny", overrides=[
        "params_dtype=bf16", "global_batch_size=4", "micro_batch_size=2", "expert_model_parallel_size=1",
        "num_experts=0", "ffn_hidden_size=256", "lora_rank=4", "lora_targets=attn+mlp", "device=cpu",
        "recompute_granularity=selective"])
    tr = Trainer(cfg)
    tr.train_step()
    assert "slab_ce_fwd_bwd" in dry and "slab_adamw" in dry
    assert dry.count("slab_adamw") == sum(1 for g in tr.engine.all_groups() if not g.frozen)


def test_poison_fill_debug_mode_walks_the_host_path(dry, monkeypatch):
    """SLAB_POISON=1 fills the dispatcher's receive regions with NaN patterns between uses (a debug aid against stale
    reads); the host side must not disturb a step."""
    monkeypatch.setenv("SLAB_POISON", "1")
    tr, d = _trainer(["recompute_granularity=selective"], {"push": True})
    assert d.poison
    tr.train_step()
    assert torch.isnan(d.scalars[0]).all() and (d.comb.view(torch.int16) == -1).all()


def test_attention_backward_binding_argument_list(dry, monkeypatch):
    from system_lab_b200.ops import attention_kernel as ak, cuda as cops
    monkeypatch.setattr(cops, "status_word", lambda dev: torch.zeros(1, dtype=torch.int32))
    monkeypatch.setattr(ak, "_ENABLED_BWD", [True])
    b, s, hq, hkv, d = 1, 128, 4, 2, 64
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    ak.attention(q, k, v, 0.125, 0).sum().backward()
    assert dry[-2:] == ["slab_attn_fwd", "slab_attn_bwd"] and qkv.grad.shape == qkv.shape
