"""The ComfyUI boundary with stand-ins (no ComfyUI, no GPU): call conventions of the attention override, pass-through
reasons, fallback after a failure, re-patching, the WanVideoWrapper wrapper (the reference's tests/test_comfyui.py)."""

import sys
import types

import pytest
import torch

import unicaattention_b200 as unica
from unicaattention_b200 import comfyui as nodes


class Patcher:
    """What the nodes use of ComfyUI's ModelPatcher."""

    def __init__(self, options=None):
        self.model_options = options if options is not None else {"transformer_options": {}}

    def clone(self):
        return Patcher({"transformer_options": dict(self.model_options["transformer_options"])})


@pytest.fixture
def fake_unica(monkeypatch):
    """unica.attention replaced by exact attention on whatever device, recording its settings; tensors claim to be on
    the GPU so that the routing rules can be exercised on the CPU."""
    calls = []

    def attention(q, k, v, **settings):
        calls.append(settings)
        return torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float()).to(q.dtype)

    monkeypatch.setattr(unica, "attention", attention)
    monkeypatch.setattr(nodes, "checked", lambda: unica.Compatibility(unica.OK, ()))
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))
    nodes.FAILED.clear()
    yield calls
    nodes.FAILED.clear()


def model_attention(q, k, v, *args, **kwargs):
    return "model's own"


def test_native_override_conventions(fake_unica):
    (patched,) = nodes.UnicaAttentionNative().patch(Patcher(), True, v_scale="per_channel")
    override = patched.model_options["transformer_options"]["optimized_attention_override"]
    q = torch.randn(2, 50, 3 * 128)
    exact = torch.nn.functional.scaled_dot_product_attention(*(x.view(2, 50, 3, 128).transpose(1, 2) for x in (q, q, q)))
    out = override(model_attention, q, q, q, heads=3)  # heads by name (WAN)
    assert out.shape == q.shape and torch.allclose(out.view(2, 50, 3, 128).transpose(1, 2), exact, atol=3e-2)
    assert fake_unica[-1] == unica.PRESETS["per_channel"]
    assert override(model_attention, q, q, q, 3).shape == q.shape  # heads by position (Flux, ...)
    bhnd = q.view(2, 50, 3, 128).transpose(1, 2)
    out = override(model_attention, bhnd, bhnd, bhnd, 3, skip_reshape=True, skip_output_reshape=True)
    assert out.shape == bhnd.shape and torch.allclose(out, exact, atol=3e-2)
    out = override(model_attention, bhnd, bhnd, bhnd, 3, skip_reshape=True)
    assert out.shape == q.shape


def test_native_override_passes_other_calls_through(fake_unica):
    (patched,) = nodes.UnicaAttentionNative().patch(Patcher(), True)
    override = patched.model_options["transformer_options"]["optimized_attention_override"]
    q = torch.randn(1, 20, 2 * 128)
    cases = [((q, q, q), dict(heads=2, mask=torch.ones(20, 20)), "mask"),
             ((q, q[:, :7], q[:, :7]), dict(heads=2), "cross-attention"),
             ((torch.randn(1, 20, 2 * 64),) * 3, dict(heads=2), "head size 64"),
             ((q, q, q), dict(), "no heads"),
             ((q, q, q), dict(heads=2, scale=0.5), "scale"),
             ((q, q, torch.randn(1, 20, 128)), dict(heads=2), "q, k, v shapes differ")]
    for tensors, kwargs, reason in cases:
        assert override(model_attention, *tensors, **kwargs) == "model's own"
        assert override.last_reason == reason
    assert not fake_unica
    assert override(model_attention, q, q, q, 2, None, None, False, False, "extra") == "model's own"
    assert override.last_reason == "positional arguments"


def test_previous_override_and_repatching(fake_unica):
    def previous(func, q, k, v, *args, **kwargs):
        return "previous override"

    model = Patcher({"transformer_options": {"optimized_attention_override": previous}})
    (once,) = nodes.UnicaAttentionNative().patch(model, True, v_scale="per_token")
    (twice,) = nodes.UnicaAttentionNative().patch(once, True, mode="fast")
    override = twice.model_options["transformer_options"]["optimized_attention_override"]
    assert override.unica and override.previous is previous  # not stacked on the first patch
    q = torch.randn(1, 20, 2 * 128)
    assert override(model_attention, q, q[:, :5], q[:, :5], heads=2) == "previous override"
    override(model_attention, q, q, q, heads=2)
    assert fake_unica[-1] == unica.PRESETS["fast"]
    first = once.model_options["transformer_options"]["optimized_attention_override"]
    first(model_attention, q, q, q, heads=2)
    assert fake_unica[-1] == unica.PRESETS["per_token"]  # each patched model keeps its own settings
    assert model.model_options["transformer_options"]["optimized_attention_override"] is previous  # the original is untouched
    (off,) = nodes.UnicaAttentionNative().patch(model, False)
    assert off is model


def test_failure_falls_back_for_good(fake_unica, monkeypatch):
    def broken(q, k, v, **settings):
        raise RuntimeError("no library")

    monkeypatch.setattr(unica, "attention", broken)
    (patched,) = nodes.UnicaAttentionNative().patch(Patcher(), True)
    override = patched.model_options["transformer_options"]["optimized_attention_override"]
    q = torch.randn(1, 20, 2 * 128)
    assert override(model_attention, q, q, q, heads=2) == "model's own" and len(nodes.FAILED) == 1
    assert override(model_attention, q, q, q, heads=2) == "model's own" and override.last_reason == "unica failed"


def test_wanvideo_wrapper_routes_modes(fake_unica):
    module = types.ModuleType("custom_nodes.wrapper.wanvideo.modules.model")
    module.attention = lambda q, k, v, *args, attention_mode="sdpa", **kwargs: f"original {attention_mode}"
    sys.modules[module.__name__] = module
    try:
        (patched,) = nodes.UnicaAttentionWanVideo().patch(Patcher(), True, v_scale="per_channel", vram_reserve_mb=2048)
        assert patched.model_options["transformer_options"]["attention_mode_override"]["mode"] == "unica_per_channel"
        assert unica.VRAM_RESERVE == 2048 * 2**20
        assert nodes.wrap_attention() == 0  # wrapped once
        q = torch.randn(1, 30, 2, 128)
        assert module.attention(q, q, q, attention_mode="sageattn") == "original sageattn"
        out = module.attention(q, q, q, attention_mode="unica_fast")
        assert out.shape == q.shape and fake_unica[-1] == unica.PRESETS["fast"]
        module.attention(q, q, q, attention_mode="unica")
        assert fake_unica[-1] == unica.PRESETS["per_token"]
        assert module.attention(q, q, q, attention_mode="unica_nonsense") == "original unica_nonsense"
        nodes.FAILED.append(RuntimeError("earlier"))
        assert module.attention(q, q, q, attention_mode="unica_fast") == "original sdpa"
    finally:
        del sys.modules[module.__name__]
        unica.VRAM_RESERVE = None


def test_mode_names_round_trip():
    for v_scale in nodes.V_SCALES:
        assert nodes.mode_settings(nodes.mode_name(v_scale, "accurate")) == unica.PRESETS[v_scale]
    assert nodes.mode_settings(nodes.mode_name("per_token", "fast")) == unica.PRESETS["fast"]
    assert nodes.mode_settings("sdpa") is None and nodes.mode_settings("unica") == unica.PRESETS["per_token"]
    assert set(nodes.NODE_CLASS_MAPPINGS) == set(nodes.NODE_DISPLAY_NAME_MAPPINGS)


class WanSelfAttention(torch.nn.Module):
    """What fused_rope_forward uses of ComfyUI's module of that name: the projections, the norms and the sizes."""

    def __init__(self, heads=2, dim=128):
        super().__init__()
        self.num_heads, self.head_dim = heads, dim
        self.q, self.k, self.v, self.o = (torch.nn.Linear(heads * dim, heads * dim) for _ in range(4))
        self.norm_q = self.norm_k = torch.nn.Identity()

    def forward(self, x, freqs, transformer_options={}):  # noqa: B006
        return "model's own forward"


class WanCrossAttention(WanSelfAttention):
    pass


class BlockPatcher(Patcher):
    """A ModelPatcher with diffusion_model.blocks and object patches."""

    def __init__(self, blocks, options=None):
        super().__init__(options)
        self.blocks, self.object_patches = blocks, {}

    def clone(self):
        return BlockPatcher(self.blocks, {"transformer_options": dict(self.model_options["transformer_options"])})

    def get_model_object(self, name):
        if name == "diffusion_model.blocks":
            return self.blocks
        return getattr(self.blocks[int(name.split(".")[2])], name.split(".")[3])

    def add_object_patch(self, name, value):
        self.object_patches[name] = value


def test_fused_rope_forward(fake_unica):
    """fuse_rope: the self-attention blocks' forward hands q, k (not rotated) and the model's table to unica; calls it
    cannot take go to the original forward (the reference's tests/test_comfyui.py covers its patch the same way)."""
    blocks = [types.SimpleNamespace(self_attn=WanSelfAttention(), cross_attn=WanCrossAttention()) for _ in range(2)]
    blocks.append(types.SimpleNamespace(self_attn=WanCrossAttention()))  # derived class in a self_attn slot: left alone
    (patched,) = nodes.UnicaAttentionNative().patch(BlockPatcher(blocks), True, v_scale="per_channel", fuse_rope=True)
    assert sorted(patched.object_patches) == [f"diffusion_model.blocks.{i}.self_attn.forward" for i in range(2)]
    forward = patched.object_patches["diffusion_model.blocks.0.self_attn.forward"]
    module = blocks[0].self_attn
    x, freqs = torch.randn(2, 50, 256), torch.zeros(1, 50, 1, 64, 2, 2)
    out = forward(x, freqs)
    assert fake_unica[-1] == unica.PRESETS["per_channel"] | {"rope": freqs}
    heads = lambda t: t.view(2, 50, 2, 128).transpose(1, 2)  # noqa: E731
    exact = torch.nn.functional.scaled_dot_product_attention(heads(module.q(x)), heads(module.k(x)), heads(module.v(x)))
    assert torch.allclose(out, module.o(exact.transpose(1, 2).reshape(2, 50, 256)), atol=3e-2)
    # what it cannot take: no table, a table of another length, an attn1 patch
    assert forward(x, None) == "model's own forward"
    assert forward(x, freqs[:, :40]) == "model's own forward"
    assert forward(x, freqs, transformer_options={"patches": {"attn1_patch": [print]}}) == "model's own forward"
    # patched again: the new forward wraps the module's own, not the first patch
    again = BlockPatcher(blocks)
    again.object_patches = dict(patched.object_patches)
    assert nodes.patch_self_attention_forward(again, unica.PRESETS["fast"]) == 2
    assert again.object_patches["diffusion_model.blocks.0.self_attn.forward"].original == module.forward
    # a failure sends this call and the later ones to the model's forward
    def broken(*args, **kwargs):
        raise RuntimeError("driver error")
    unica.attention = broken  # the fixture's monkeypatch restores it
    assert forward(x, freqs) == "model's own forward" and nodes.FAILED
    assert forward(x, freqs) == "model's own forward"


def test_measurement_count_runs_per_step_and_block():
    """The count is step * blocks + block + 1 within a run; calls outside the numbered blocks are not counted once the
    model is known to number its blocks; a model that numbers none is counted call by call; off, nothing is read
    (the reference's tests/test_comfyui.py:114-140)."""
    m = nodes.Measurement("test")
    m.every = 1000  # counting runs only while measuring
    sigma = lambda s: {"sigmas": torch.tensor([s])}  # noqa: E731
    seen = []
    for s in (1.0, 0.5):  # two steps of a 3-block model, each preceded by a refiner call
        m.due(sigma(s))
        for block in range(3):
            m.due(sigma(s) | {"block_index": block, "total_blocks": 3})
            seen.append(m.calls)
    assert seen == [1, 2, 3, 4, 5, 6], seen
    m.due(sigma(1.0) | {"block_index": 0, "total_blocks": 3})  # sigma rises: a new run
    assert m.calls == 1
    plain = nodes.Measurement("test")
    plain.every = 2
    assert [plain.due(sigma(1.0)) for _ in range(4)] == [False, True, False, True]

    class Untouchable:
        def max(self):
            raise AssertionError("sigma read while not measuring")

    assert not nodes.Measurement("test").due({"sigmas": Untouchable(), "block_index": 0})


def test_measurement_writes_a_row_per_measured_call(fake_unica, tmp_path, monkeypatch):
    """Every second call of the native node is measured: one CSV row with the error of the call as it ran and of every
    preset against FP32, the input statistics and the routes; with the flag file present the tensors are dumped too."""
    import csv

    monkeypatch.setenv("UNICA_MEASURE_DIR", str(tmp_path))
    monkeypatch.delenv("UNICA_EMULATOR", raising=False)
    (patched,) = nodes.UnicaAttentionNative().patch(Patcher(), True, v_scale="per_channel", measure_every=2, measure_heads=2,
                                                    measure_tag="stand-in")
    override = patched.model_options["transformer_options"]["optimized_attention_override"]
    q = torch.randn(1, 40, 3 * 128)
    override(model_attention, q, q, q, heads=3)
    assert not (tmp_path / "attention_errors.csv").exists()
    (tmp_path / "dumps.flag").touch()
    override(model_attention, q, q[:, :7], q[:, :7], heads=3)  # passed on: counted as a route, not as a call
    override(model_attention, q, q, q, heads=3)
    with (tmp_path / "attention_errors.csv").open() as f:
        rows = list(csv.DictReader(f))
    assert len(rows) == 1 and rows[0]["tag"] == "stand-in" and rows[0]["ran"] == "per_channel" and rows[0]["call"] == "2"
    assert rows[0]["heads_measured"] == "2" and rows[0]["tokens"] == "40" and "cross-attention=1" in rows[0]["routes"]
    assert float(rows[0]["unica_rel_l2"]) < 0.05 and float(rows[0]["fast_rel_l2"]) < 0.05  # the stand-in is exact up to bf16
    assert rows[0]["emulated_fast_rel_l2"] == "" and float(rows[0]["q_channel_spread"]) > 1
    dumps = list((tmp_path / "dumps").glob("*.pt"))
    assert len(dumps) == 1 and torch.load(dumps[0])["q"].shape == (1, 2, 40, 128)
    nodes.native_measurement.configure(0, 0)
