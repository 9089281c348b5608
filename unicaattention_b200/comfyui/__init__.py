"""ComfyUI nodes that run a model's self-attention on unicaattention_b200: the drop-in boundary of the reference's
comfyui/__init__.py (same node classes, inputs, override call convention, routing rules, fallback, fused-RoPE forward
and measurement mode, see measure.py), without its SageAttention comparison and RIFE node.

    model -> Unica Attention (native)   -> sampler     ComfyUI's own models: an `optimized_attention_override`
    WanVideoModelLoader -> Unica Attention (WanVideo) -> WanVideoSampler   ComfyUI-WanVideoWrapper: `attention` wrapped

Routing (comfyui/__init__.py:379-409 in the reference): only self-attention with head_dim 128, as many keys as queries,
q, k, v of one shape, no mask, the default scale, on the GPU goes to unica; every other call goes to the override that
was on the model before, or to the function ComfyUI passed.  The first unica call that raises one of `UNICA_ERRORS` is
logged and sends that call and every later one back to the model's own attention.

ComfyUI itself is not imported here: the nodes only touch `model.clone()` and `model_options`, so tests drive them
with stand-ins.
"""

from __future__ import annotations

import functools
import logging
import sys

import torch

import unicaattention_b200 as unica
from unicaattention_b200.comfyui.measure import Measurement

HEAD_DIM = 128
MODE = "unica"  # WanVideoWrapper attention modes: "unica" (per token), "unica_<v_scale>", "unica_fast"
log = logging.getLogger("UnicaAttention")

V_SCALES = {name: unica.PRESETS[name] for name in ("per_token", "outliers", "per_channel")}
FAST = unica.PRESETS["fast"]
# positional parameters of ComfyUI's attention functions after q, k, v (comfy/ldm/modules/attention.py)
POSITIONAL = ("heads", "mask", "attn_precision", "skip_reshape", "skip_output_reshape")
# what unica.attention raises for a call it cannot take (its checks) or cannot run (the library, the driver)
UNICA_ERRORS = (RuntimeError, ValueError, TypeError)
FAILED: list = []  # the first error, once a call has failed: from then on nothing is routed to unica
measurement = Measurement("WanVideo")  # off until a node's measure_every input turns it on
native_measurement = Measurement("native")
MEASURE_INPUTS = {
    "measure_every": ("INT", {"default": 0, "min": 0, "max": 100000,
                              "tooltip": "Run every n-th self-attention call again with every preset and in FP32, and write "
                                         "the errors to a CSV (0: off)"}),
    "measure_heads": ("INT", {"default": 2, "min": 1, "max": 40, "tooltip": "Heads per measured call: the FP32 reference is slow"}),
    "measure_tag": ("STRING", {"default": "", "tooltip": "Written into the measurement CSV, e.g. the model's name"}),
}


def unica_nhd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, settings: dict) -> torch.Tensor:
    """unica.attention on [batch, tokens, heads, 128] tensors of any float dtype.  bf16 and fp16 are read through a
    transposed view and the output comes back in the same layout, without copies; float32 is converted once each way."""
    half = q.dtype if q.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
    out = unica.attention(*(x.transpose(1, 2).to(half) for x in (q, k, v)), **settings)
    return out.transpose(1, 2).to(q.dtype).contiguous()


@functools.cache
def checked() -> unica.Compatibility:
    """unica.compatibility(), logged once; on a machine that cannot run the library the nodes leave models untouched."""
    status = unica.compatibility()
    if status.status != unica.OK:
        log.warning("%s%s", status, "\nThe Unica nodes leave the model's own attention in place."
                    if status.status == unica.UNSUPPORTED else "")
    return status


# ----------------------------------------------------------------------------------------------------------------------
# settings <-> node inputs <-> WanVideoWrapper mode names


def choose_kernel(v_scale: str, mode: str, vram_reserve_mb: int) -> dict:
    """The keyword arguments unica.attention gets for a node's inputs.  The VRAM reserve belongs to the machine, not to
    a model: the node that ran last sets it for every call."""
    unica.VRAM_RESERVE = vram_reserve_mb * 2**20 if vram_reserve_mb else None
    return FAST if mode == "fast" else V_SCALES[v_scale]


def mode_name(v_scale: str, mode: str) -> str:
    return f"{MODE}_fast" if mode == "fast" else f"{MODE}_{v_scale}"


def mode_settings(attention_mode: str) -> dict | None:
    """Settings of a WanVideoWrapper attention mode, None when the mode is not one of unica's."""
    if attention_mode == MODE:
        return V_SCALES["per_token"]
    if not attention_mode.startswith(MODE + "_"):
        return None
    name = attention_mode[len(MODE) + 1:]
    return FAST if name == "fast" else V_SCALES.get(name)


KERNEL_INPUTS = {
    "v_scale": (list(V_SCALES), {"default": "per_token",
                                 "tooltip": "V's INT8 scale in the accurate mode: per token (folded into P), outliers (per "
                                            "channel without each head's 8 largest keys, added exactly) or per channel"}),
    "vram_reserve_mb": ("INT", {"default": 0, "min": 0, "max": 65536, "step": 64,
                                "tooltip": "VRAM left free for other programs; 0: the larger of 1 GiB and a tenth of the "
                                           "card.  A call that would reach it runs a few heads at a time"}),
    "mode": (["accurate", "fast"], {"default": "accurate",
                                    "tooltip": "accurate: INT8 Q.K^T and u8 x s8 P.V.  fast: NVFP4 for both, Q smoothed per "
                                               "512 queries; v_scale does not apply"}),
}


# ----------------------------------------------------------------------------------------------------------------------
# ComfyUI's own models: optimized_attention_override


def pass_through_reason(q, k, v, args: tuple, named: dict) -> str | None:
    """Why a call is not unica's, or None if it is."""
    if FAILED:
        return "unica failed"
    if len(args) > len(POSITIONAL):
        return "positional arguments"
    heads = named.get("heads")
    if heads is None:
        return "no heads"
    if named.get("mask") is not None:
        return "mask"
    if not q.is_cuda:
        return "not on the GPU"
    by_head = named.get("skip_reshape", False)  # [batch, heads, tokens, dim] instead of [batch, tokens, heads * dim]
    dim = q.shape[-1] if by_head else q.shape[-1] // heads
    token_axis = 2 if by_head else 1
    if dim != HEAD_DIM:
        return f"head size {dim}"
    if k.shape[token_axis] != q.shape[token_axis]:
        return "cross-attention"
    if not q.shape == k.shape == v.shape:
        return "q, k, v shapes differ"
    if named.get("scale") not in (None, HEAD_DIM**-0.5):
        return "scale"
    return None


def native_override(previous, settings: dict):
    """An `optimized_attention_override`: ComfyUI calls it as (func, q, k, v, heads=..., ...) with q, k, v
    [batch, tokens, heads * dim], or [batch, heads, tokens, dim] with skip_reshape.  `previous`: the override that was on
    the model (or None); it, or func, gets every call that is not unica's."""

    def elsewhere(func, q, k, v, args, kwargs):
        return previous(func, q, k, v, *args, **kwargs) if previous else func(q, k, v, *args, **kwargs)

    def override(func, q, k, v, *args, **kwargs):
        named = dict(zip(POSITIONAL, args)) | kwargs  # WAN passes heads by name, most other models by position
        override.last_reason = pass_through_reason(q, k, v, args, named)
        native_measurement.route(override.last_reason, q, k)
        if override.last_reason is not None:
            return elsewhere(func, q, k, v, args, kwargs)
        heads = named["heads"]
        by_head, keep_heads = named.get("skip_reshape", False), named.get("skip_output_reshape", False)
        nhd = [x.transpose(1, 2) if by_head else x.view(x.shape[0], x.shape[1], heads, HEAD_DIM) for x in (q, k, v)]
        try:
            out = unica_nhd(*nhd, settings)
        except UNICA_ERRORS as error:
            if not FAILED:
                log.error("unica failed, the model's own attention takes over: %s", error)
            FAILED.append(error)
            return elsewhere(func, q, k, v, args, kwargs)
        native_measurement(*nhd, settings, options=named.get("transformer_options"))
        return out.transpose(1, 2) if keep_heads else out.reshape(out.shape[0], out.shape[1], heads * HEAD_DIM)

    override.unica, override.previous, override.last_reason = True, previous, None
    return override


def fused_rope_forward(module, original, settings: dict):
    """A forward for ComfyUI's WanSelfAttention that hands q and k to unica BEFORE RoPE, with the model's own table: the
    quantizers rotate them on the way in, so the model's pass over q and k to rotate them goes, and with it a bf16
    rounding (comfyui/__init__.py:415-441 in the reference).  The rest as the module does it: q = norm_q(q(x)),
    k = norm_k(k(x)), v = v(x), out = o(attention).  Calls with an attn1_patch (it wants the rotated q and k), another
    head size, no table or a table that does not fit, tensors off the GPU, and every call after a failure go to the
    original forward."""

    def forward(x, freqs, transformer_options={}):  # noqa: B006 (the signature of the forward it replaces)
        batch, tokens, heads, dim = *x.shape[:2], module.num_heads, module.head_dim
        if (FAILED or transformer_options.get("patches", {}).get("attn1_patch") or freqs is None or dim != HEAD_DIM
                or not x.is_cuda or freqs.dim() != 6 or freqs.shape[1] != tokens):
            return original(x, freqs, transformer_options=transformer_options)
        q = module.norm_q(module.q(x)).view(batch, tokens, heads, dim)
        k = module.norm_k(module.k(x)).view(batch, tokens, heads, dim)
        v = module.v(x).view(batch, tokens, heads, dim)
        try:
            half = q.dtype if q.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
            out = unica.attention(*(t.transpose(1, 2).to(half) for t in (q, k, v)), rope=freqs, **settings)
        except UNICA_ERRORS as error:
            log.error("unica failed, the model's own attention takes over: %s", error)
            FAILED.append(error)
            return original(x, freqs, transformer_options=transformer_options)
        return module.o(out.transpose(1, 2).reshape(batch, tokens, heads * dim).to(x.dtype))

    forward.unica, forward.original = True, original
    return forward


def patch_self_attention_forward(patched, settings: dict) -> int:
    """fused_rope_forward on every WanSelfAttention of the model, as object patches of this clone only; returns how
    many.  Cross-attention classes derive from WanSelfAttention and are left alone."""
    blocks = patched.get_model_object("diffusion_model.blocks")
    count = 0
    for i in range(len(blocks)):
        name = f"diffusion_model.blocks.{i}.self_attn"
        module = patched.get_model_object(name)
        if type(module).__name__ != "WanSelfAttention":
            continue
        original = patched.object_patches.get(f"{name}.forward", module.forward)
        if getattr(original, "unica", False):  # patched before: wrap what was there before it
            original = original.original
        patched.add_object_patch(f"{name}.forward", fused_rope_forward(module, original, settings))
        count += 1
    return count


class UnicaAttentionNative:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("MODEL",),
                             "enabled": ("BOOLEAN", {"default": True, "tooltip": "Off: the model as it came, for A/B runs"})},
                "optional": dict(KERNEL_INPUTS) | MEASURE_INPUTS | {
                    "fuse_rope": ("BOOLEAN", {"default": False,
                                              "tooltip": "WAN models: rotate q and k inside the quantization instead of "
                                                         "in a pass of their own before attention"})}}

    RETURN_TYPES = ("MODEL",)
    RETURN_NAMES = ("model",)
    FUNCTION = "patch"
    CATEGORY = "UnicaAttention"
    DESCRIPTION = ("Self-attention on unica-b200 through optimized_attention_override.  Put it after other attention "
                   "patches: calls it does not take (cross-attention, masks) go to the override before it.")

    def patch(self, model, enabled, v_scale="per_token", mode="accurate", vram_reserve_mb=0, fuse_rope=False, measure_every=0,
              measure_heads=2, measure_tag="", **ignored):
        if not enabled or checked().status == unica.UNSUPPORTED:
            return (model,)
        settings = choose_kernel(v_scale, mode, vram_reserve_mb)
        native_measurement.configure(measure_every, measure_heads, measure_tag)
        native_measurement.routes.clear()
        native_measurement.sigma, native_measurement.numbered = None, False  # a new model starts its own count
        patched = model.clone()
        options = patched.model_options.setdefault("transformer_options", {})
        previous = options.get("optimized_attention_override")
        if getattr(previous, "unica", False):  # patched before: wrap what was there before it, with the new settings
            previous = previous.previous
        options["optimized_attention_override"] = native_override(previous, settings)
        if fuse_rope and not patch_self_attention_forward(patched, settings):
            log.warning("fuse_rope: the model has no WanSelfAttention blocks; nothing fused")
        return (patched,)


# ----------------------------------------------------------------------------------------------------------------------
# ComfyUI-WanVideoWrapper: its `attention` function, wrapped once per loaded model module


def wrap_attention() -> int:
    """Wraps `attention` in every loaded `*.wanvideo.modules.model` module, once; returns how many it wrapped."""
    wrapped = 0
    for name, module in list(sys.modules.items()):
        original = getattr(module, "attention", None)
        if not name.endswith("wanvideo.modules.model") or original is None or getattr(original, "unica", False):
            continue

        def attention(q, k, v, *args, attention_mode="sdpa", original=original, **kwargs):
            settings = mode_settings(attention_mode)
            if settings is None:
                return original(q, k, v, *args, attention_mode=attention_mode, **kwargs)
            if not FAILED:
                try:
                    out = unica_nhd(q, k, v, settings)
                    measurement(q, k, v, settings)
                    return out
                except UNICA_ERRORS as error:
                    log.error("unica failed, sdpa takes over: %s", error)
                    FAILED.append(error)
            return original(q, k, v, *args, attention_mode="sdpa", **kwargs)

        attention.unica = True
        module.attention = attention
        wrapped += 1
    return wrapped


def _wrapped_already() -> bool:
    return any(getattr(getattr(m, "attention", None), "unica", False)
               for n, m in sys.modules.items() if n.endswith("wanvideo.modules.model"))


class UnicaAttentionWanVideo:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("WANVIDEOMODEL",),
                             "enabled": ("BOOLEAN", {"default": True, "tooltip": "Off: the model as it came, for A/B runs"})},
                "optional": dict(KERNEL_INPUTS) | MEASURE_INPUTS}

    RETURN_TYPES = ("WANVIDEOMODEL",)
    RETURN_NAMES = ("model",)
    FUNCTION = "patch"
    CATEGORY = "UnicaAttention"
    DESCRIPTION = "Self-attention of a WanVideoWrapper model on unica-b200 (attention mode override)"

    def patch(self, model, enabled, v_scale="per_token", mode="accurate", vram_reserve_mb=0, measure_every=0, measure_heads=2,
              measure_tag="", **ignored):
        if not enabled or checked().status == unica.UNSUPPORTED:
            return (model,)
        choose_kernel(v_scale, mode, vram_reserve_mb)  # sets the VRAM reserve; the settings travel in the mode's name
        measurement.configure(measure_every, measure_heads, measure_tag)
        if not wrap_attention() and not _wrapped_already():
            raise RuntimeError("ComfyUI-WanVideoWrapper's wanvideo.modules.model is not loaded")
        patched = model.clone()
        patched.model_options.setdefault("transformer_options", {})["attention_mode_override"] = {
            "mode": mode_name(v_scale, mode), "start_step": 0, "end_step": 10000, "verbose": False}
        return (patched,)


NODE_CLASS_MAPPINGS = {"UnicaAttentionWanVideo": UnicaAttentionWanVideo, "UnicaAttentionNative": UnicaAttentionNative}
NODE_DISPLAY_NAME_MAPPINGS = {"UnicaAttentionWanVideo": "Unica Attention (WanVideo)",
                              "UnicaAttentionNative": "Unica Attention (native)"}
