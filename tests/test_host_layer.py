"""Host-side mirror of the node pack's interface, exercised on CPU with the fake `comfy` package.

Covers what needs no GPU: the node / ops surface saved workflows depend on, state-dict loading
branches, patcher hooks, scale slicing for fused-QKV offsets, dynamic-LoRA composition, and the
loud failure when a quantised path is asked to run without CUDA.
"""
import types

import pytest
import torch
from torch import nn

import comfy.sd
import comfy.utils
import folder_paths


@pytest.fixture()
def ops(pkg):
    o = pkg.Int8TensorwiseOps
    saved = (o.excluded_names, o.dynamic_quantize, o.enable_quarot, o._is_prequantized)
    yield o
    o.excluded_names, o.dynamic_quantize, o.enable_quarot, o._is_prequantized = saved


def load(layer, **tensors):
    sd = dict(tensors)
    missing = []
    layer._load_from_state_dict(sd, "", {}, True, missing, [], [])
    return sd, missing


def test_node_surface_matches_saved_workflows(pkg):
    assert list(pkg.NODE_CLASS_MAPPINGS) == ["OTUNetLoaderW8A8", "INT8LoraLoader", "INT8LoraLoaderStack",
                                             "INT8DynamicLoraLoader", "INT8DynamicLoraStack"]
    assert pkg.NODE_DISPLAY_NAME_MAPPINGS["OTUNetLoaderW8A8"] == "Load Diffusion Model INT8 (W8A8)"
    folder_paths.FILES["loras"] = ["a.safetensors"]
    folder_paths.FILES["diffusion_models"] = ["m.safetensors"]
    for node in pkg.NODE_CLASS_MAPPINGS.values():
        assert node.RETURN_TYPES == ("MODEL",) and node.CATEGORY == "loaders" and isinstance(node.FUNCTION, str)
        assert hasattr(node(), node.FUNCTION)
    req = pkg.NODE_CLASS_MAPPINGS["OTUNetLoaderW8A8"].INPUT_TYPES()["required"]
    assert list(req) == ["unet_name", "weight_dtype", "model_type", "on_the_fly_quantization", "enable_quarot"]
    assert req["weight_dtype"][0] == ["default", "fp8_e4m3fn", "fp16", "bf16"]
    assert req["model_type"][0] == ["flux2", "z-image", "chroma", "wan", "ltx2", "qwen", "ernie", "anima"]
    assert req["on_the_fly_quantization"][1]["default"] is False and req["enable_quarot"][1]["default"] is False
    lora = pkg.NODE_CLASS_MAPPINGS["INT8LoraLoader"].INPUT_TYPES()["required"]
    assert list(lora) == ["model", "lora_name", "strength"]
    assert (lora["strength"][1]["min"], lora["strength"][1]["max"], lora["strength"][1]["step"]) == (-10.0, 10.0, 0.01)
    dyn = pkg.NODE_CLASS_MAPPINGS["INT8DynamicLoraLoader"].INPUT_TYPES()["required"]
    assert (dyn["strength"][1]["min"], dyn["strength"][1]["max"]) == (-20.0, 20.0)
    stack = pkg.NODE_CLASS_MAPPINGS["INT8LoraLoaderStack"].INPUT_TYPES()
    assert list(stack["optional"]) == [f"{k}_{i}" for i in range(1, 11) for k in ("lora", "strength")]
    assert stack["optional"]["lora_1"][0][0] == "None"


def test_layout_registration(pkg):
    import comfy.quant_ops as qo
    algo = qo.QUANT_ALGOS["int8_tensorwise"]
    assert algo["storage_t"] == torch.int8 and algo["parameters"] == {"weight_scale", "input_scale"}
    layout = qo.LAYOUTS[algo["comfy_tensor_layout"]]
    q = torch.tensor([[1, -2]], dtype=torch.int8)
    p = layout.Params(scale=torch.tensor(0.5), orig_dtype=torch.bfloat16, orig_shape=(1, 2))
    assert torch.equal(layout.dequantize(q, p), torch.tensor([[0.5, -1.0]]))
    assert set(layout.state_dict_tensors(q, p)) == {"", "weight_scale"}
    assert p.clone().scale is not p.scale


def test_ops_class_exposes_all_layer_types(ops):
    for name in ("Linear", "GroupNorm", "LayerNorm", "Conv2d", "Conv3d", "ConvTranspose2d", "Embedding"):
        assert isinstance(getattr(ops, name), type)
    assert isinstance(ops.conv_nd(2, 4, 4, 3), ops.Conv2d) and isinstance(ops.conv_nd(3, 4, 4, 3), ops.Conv3d)
    with pytest.raises(ValueError):
        ops.conv_nd(1, 4, 4, 3)
    assert ops.use_triton is True  # accepted for compatibility


def test_load_prequantized_variants(ops):
    w = torch.randint(-100, 100, (24, 32), dtype=torch.int8)
    lin = ops.Linear(32, 24, bias=True)
    sd, missing = load(lin, weight=w, weight_scale=torch.tensor(0.0125), input_scale=torch.tensor(1.0),
                       comfy_quant=torch.zeros(1), bias=torch.zeros(24))
    assert not sd and not missing
    assert lin._is_quantized and not lin._is_per_row and lin.weight_scale is None
    assert lin._get_weight_scale() == pytest.approx(0.0125) and isinstance(lin._get_weight_scale(), float)
    assert ops._is_prequantized and lin.weight_comfy_model_dtype == torch.int8
    lin = ops.Linear(32, 24, bias=False)
    load(lin, weight=w, weight_scale=torch.rand(24, 1).half())
    assert lin._is_per_row and lin._get_weight_scale().dtype == torch.float32 and lin.bias is None
    lin = ops.Linear(32, 24, bias=False)
    load(lin, weight=w, weight_scale=torch.rand(24))
    assert lin._is_quantized and not lin._is_per_row and lin._get_weight_scale().numel() == 24
    lin = ops.Linear(32, 24)
    _, missing = load(lin)
    assert missing == ["weight"]


def test_float_weights_stay_float_unless_dynamic_quantize(ops):
    w = torch.randn(24, 32).bfloat16()
    lin = ops.Linear(32, 24, bias=False)
    load(lin, weight=w)
    assert not lin._is_quantized and lin.weight.dtype == torch.bfloat16
    y = lin(torch.randn(3, 32).bfloat16())
    assert y.shape == (3, 24)
    ops.dynamic_quantize = True
    ops.excluded_names = ["img_in"]
    lin = ops.Linear(32, 24, bias=False)
    sd = {"img_in.weight": w}
    lin._load_from_state_dict(sd, "img_in.", {}, True, [], [], [])
    assert not lin._is_quantized                      # excluded by name
    lin = ops.Linear(24, 24, bias=False)               # K not a multiple of 16: cannot feed the TMA path
    load(lin, weight=torch.randn(24, 24))
    assert not lin._is_quantized
    if not torch.cuda.is_available():
        lin = ops.Linear(32, 24, bias=False)
        with pytest.raises(RuntimeError, match="CUDA"):
            load(lin, weight=w)


def test_quantized_forward_refuses_cpu(ops, pkg):
    lin = ops.Linear(32, 24, bias=False)
    load(lin, weight=torch.zeros(24, 32, dtype=torch.int8), weight_scale=torch.tensor(0.1))
    with pytest.raises(pkg._native.NativeLibraryError, match="CUDA"):
        lin(torch.zeros(40, 32, dtype=torch.bfloat16))


def test_patcher_hooks(ops):
    w = torch.randint(-100, 100, (24, 32), dtype=torch.int8)
    lin = ops.Linear(32, 24, bias=True)
    load(lin, weight=w, weight_scale=torch.tensor(0.5), bias=torch.zeros(24))
    assert lin.convert_weight(torch.zeros(1)) is lin.weight
    new = torch.ones(24, 32, dtype=torch.int8)
    assert lin.set_weight(new, return_weight=True) is new
    lin.set_weight(new, inplace_update=True)
    assert torch.equal(lin.weight, new)
    lin.set_weight(new * 2)
    assert torch.equal(lin.weight, new * 2) and not lin.weight.requires_grad
    assert lin.set_bias(None) is None
    lin.set_bias(torch.ones(24), inplace_update=True)
    assert torch.equal(lin.bias, torch.ones(24))
    flt = ops.Linear(32, 24, bias=False)
    load(flt, weight=torch.randn(24, 32).half())
    assert flt.convert_weight("x") == "x"
    flt.set_weight(torch.ones(24, 32))
    assert flt.weight.dtype == torch.float16


def test_scale_slicing_for_fused_qkv(pkg):
    o = pkg.ops
    ws = torch.arange(12.0).reshape(12, 1)
    assert o._slice_scale(0.5, 4, (0, 4, 4)) == 0.5
    assert torch.equal(o._slice_scale(ws, 4, (0, 4, 4)), ws[4:8])
    assert torch.equal(o._slice_scale(ws, 4, (0, 10, 4)), ws[10:12])       # clipped to what exists
    assert torch.equal(o._slice_scale(ws, 4, None), ws[:4])                # unknown chunk: first rows
    assert torch.equal(o._slice_scale(ws, 12, None), ws)
    assert torch.equal(o._slice_scale_strict(ws, 4, (0, 8, 4)), ws[8:12])
    assert torch.equal(o._slice_scale_strict(ws, 12, (0, 8, 4)), ws)


def test_reconstruct_lora_diff_kinds(pkg):
    o = pkg.ops
    up, down = torch.randn(6, 2), torch.randn(2, 8)
    d, s = o.reconstruct_lora_diff((up, down, 4.0, None, None, None), (6, 8), "cpu", torch.float32, 0.5)
    assert torch.allclose(d, up @ down) and s == pytest.approx(4.0 / 2 * 0.5)
    mid = torch.randn(2, 2)
    d, s = o.reconstruct_lora_diff((up, down, None, mid, None, None), (6, 8), "cpu", torch.float32, 0.5)
    assert torch.allclose(d, up @ (mid @ down)) and s == 0.5
    w1a, w1b, w2a, w2b = torch.randn(6, 2), torch.randn(2, 8), torch.randn(6, 2), torch.randn(2, 8)
    d, s = o.reconstruct_lora_diff((w1a, w1b, 2.0, w2a, w2b, None, None, None), (6, 8), "cpu", torch.float32, 1.0)
    assert torch.allclose(d, (w1a @ w1b) * (w2a @ w2b)) and s == 1.0
    w1, w2 = torch.randn(2, 2), torch.randn(3, 4)
    d, s = o.reconstruct_lora_diff((w1, w2, None, None, None, None, None, None, None), (6, 8), "cpu", torch.float32, 2.0)
    assert torch.allclose(d, torch.kron(w1, w2)) and s == 2.0
    assert o.reconstruct_lora_diff((1, 2, 3), (6, 8), "cpu", torch.float32, 1.0) == (None, 1.0)


class _Block(nn.Module):
    def __init__(self, ops):
        super().__init__()
        self.qkv = ops.Linear(32, 48, bias=False)
        self.proj = ops.Linear(32, 32, bias=False)


class _Diffusion(nn.Module):
    def __init__(self, ops):
        super().__init__()
        self.blocks = nn.ModuleList([_Block(ops), _Block(ops)])
        self.img_in = ops.Linear(32, 32, bias=False)

    def forward(self, x, t=None, context=None, transformer_options=None):
        return x


class _Patcher:
    def __init__(self, diffusion):
        self.model = types.SimpleNamespace(diffusion_model=diffusion, model_type=types.SimpleNamespace(name="FLUX"))
        self.model_options = {}
        self.patches = []

    def clone(self):
        c = _Patcher(self.model.diffusion_model)
        c.model_options = {k: (dict(v) if isinstance(v, dict) else v) for k, v in self.model_options.items()}
        c.patches = list(self.patches)
        return c

    def add_patches(self, patches, strength):
        self.patches.append((patches, strength))


def _quantized_model(ops):
    m = _Diffusion(ops)
    for mod in m.modules():
        if isinstance(mod, ops.Linear) and mod is not m.img_in:
            load(mod, weight=torch.zeros(mod.out_features, mod.in_features, dtype=torch.int8),
                 weight_scale=torch.rand(mod.out_features, 1) + 0.1)
    load(m.img_in, weight=torch.zeros(32, 32).half())
    return m


def _lora_file(name, targets, rank=4):
    state = {}
    for prefix, (n, k) in targets.items():
        state[f"{prefix}.lora_up.weight"] = torch.randn(n, rank)
        state[f"{prefix}.lora_down.weight"] = torch.randn(rank, k)
        state[f"{prefix}.alpha"] = torch.tensor(2.0)
    comfy.utils.FILES[f"/loras/{name}"] = state


def test_dynamic_lora_nodes_compose_factors(ops, pkg):
    model = _Patcher(_quantized_model(ops))
    _lora_file("a", {"diffusion_model.blocks.0.qkv": (48, 32), "diffusion_model.blocks.1.proj": (32, 32)})
    _lora_file("b", {"diffusion_model.blocks.0.qkv": (48, 32)}, rank=2)
    node = pkg.NODE_CLASS_MAPPINGS["INT8DynamicLoraStack"]()
    (out,) = node.apply_stack(model, lora_1="a", strength_1=0.5, lora_2="b", strength_2=2.0, lora_3="None", strength_3=1.0)
    assert out is not model and "transformer_options" not in model.model_options
    loras = out.model_options["transformer_options"]["dynamic_loras"]
    assert [d["name"] for d in loras] == ["a", "b"] and [d["strength"] for d in loras] == [0.5, 2.0]
    dm = out.model.diffusion_model
    hook = dm._dynamic_lora_hook
    assert pkg.ops.DynamicLoRAHook.register(dm) is hook          # registered once
    hook.pre_forward(dm, (), {"transformer_options": out.model_options["transformer_options"]})
    qkv = dm.blocks[0].qkv
    assert qkv.lora_A.shape == (6, 32) and qkv.lora_B.shape == (48, 6) and qkv.lora_alpha is None
    a_state, b_state = comfy.utils.FILES["/loras/a"], comfy.utils.FILES["/loras/b"]
    want_a = torch.cat([a_state["diffusion_model.blocks.0.qkv.lora_down.weight"] * (2.0 / 4 * 0.5),
                        b_state["diffusion_model.blocks.0.qkv.lora_down.weight"] * (2.0 / 2 * 2.0)])
    assert torch.allclose(qkv.lora_A, want_a)
    assert dm.blocks[1].proj.lora_A.shape == (4, 32) and dm.blocks[1].qkv.lora_A is None
    first_id = hook.current_lora_id
    hook.pre_forward(dm, (), {"transformer_options": out.model_options["transformer_options"]})
    assert hook.current_lora_id == first_id
    hook.pre_forward(dm, (None, None, {"transformer_options": {}}), {})      # options passed positionally, no LoRAs
    assert qkv.lora_A is None and qkv.lora_B is None
    (same,) = pkg.NODE_CLASS_MAPPINGS["INT8DynamicLoraLoader"]().load_lora(model, "a", 0)
    assert same is model


def test_stochastic_lora_nodes_upgrade_adapters(ops, pkg):
    model = _Patcher(_quantized_model(ops))
    _lora_file("a", {"diffusion_model.blocks.0.qkv": (48, 32), "diffusion_model.img_in": (32, 32)})
    (out,) = pkg.NODE_CLASS_MAPPINGS["INT8LoraLoader"]().load_lora(model, "a", 0.8)
    (patches, strength), = out.patches
    assert strength == 0.8 and not model.patches
    quant = patches["diffusion_model.blocks.0.qkv.weight"]
    assert isinstance(quant, pkg.ops.INT8LoRAPatchAdapter) and quant.seed == 318008
    assert torch.equal(quant.weight_scale, model.model.diffusion_model.blocks[0].qkv.weight_scale)
    assert type(patches["diffusion_model.img_in.weight"]).__name__ == "LoRAAdapter"   # float layer keeps the stock adapter
    _lora_file("b", {"diffusion_model.blocks.0.qkv": (48, 32)})
    (out,) = pkg.NODE_CLASS_MAPPINGS["INT8LoraLoaderStack"]().apply_stack(model, lora_1="a", strength_1=1.0, lora_2="b",
                                                                         strength_2=-0.5)
    (patches, strength), = out.patches
    merged = patches["diffusion_model.blocks.0.qkv.weight"]
    assert strength == 1.0 and isinstance(merged, pkg.ops.INT8MergedLoRAPatchAdapter)
    assert [s for _, s in merged.patches] == [1.0, -0.5]
    assert patches["diffusion_model.img_in.weight"].weight_scale == 1.0
    (same,) = pkg.NODE_CLASS_MAPPINGS["INT8LoraLoaderStack"]().apply_stack(model)
    assert same is model


def test_loader_node_sets_class_flags(ops, pkg):
    seen = {}

    def fake_loader(path, model_options):
        seen.update(path=path, ops=model_options["custom_operations"])
        return "MODEL"
    comfy.sd.LOADER = fake_loader
    node = pkg.NODE_CLASS_MAPPINGS["OTUNetLoaderW8A8"]()
    assert node.load_unet("m.safetensors", "default", "flux2", True, True) == ("MODEL",)
    assert seen["path"] == "/diffusion_models/m.safetensors" and seen["ops"] is ops
    assert ops.dynamic_quantize is True and ops.enable_quarot is True and ops._is_prequantized is False
    assert "double_stream_modulation_img" in ops.excluded_names and "img_in" in ops.excluded_names
    node.load_unet("m.safetensors", "default", "wan", False)
    assert ops.excluded_names == ["patch_embedding", "text_embedding", "time_embedding", "time_projection", "head", "img_emb"]
    assert ops.dynamic_quantize is False and ops.enable_quarot is False


def test_build_hadamard_matches_sylvester(pkg):
    h = pkg.quarot.build_hadamard(128)
    assert torch.allclose(h @ h.T, torch.eye(128), atol=1e-6)
    assert h[0, 0] > 0 and torch.allclose(h[1, :4] * (128 ** 0.5), torch.tensor([1.0, -1.0, 1.0, -1.0]))
    with pytest.raises(ValueError):
        pkg.quarot.build_hadamard(96)


def test_custom_ops_have_shape_functions(pkg):
    """The registered operators carry fake kernels, so tracing sees one node with a known output shape."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    assert pkg.custom_ops.linear_forward is not None
    with FakeTensorMode():
        x = torch.empty(40, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(24, 64, dtype=torch.int8, device="cuda")
        ws = torch.empty(24, dtype=torch.float32, device="cuda")
        y = torch.ops.int8_fast_b200.linear_forward(x, w, ws, None, torch.bfloat16, True, 0)
        assert y.shape == (40, 24) and y.dtype == torch.bfloat16 and y.device.type == "cuda"
        a = torch.empty(8, 64, dtype=torch.bfloat16, device="cuda")
        b = torch.empty(24, 8, dtype=torch.bfloat16, device="cuda")
        y2 = torch.ops.int8_fast_b200.linear_lora_forward(x, w, ws, None, a, b, torch.float16, False, True, 0)
        assert y2.shape == (40, 24) and y2.dtype == torch.float16
        y3 = torch.ops.int8_fast_b200.small_batch_forward(x[:4], w, ws, None, a, b, False)
        assert y3.shape == (4, 24) and y3.dtype == torch.bfloat16


def test_lora_cache_follows_the_source_tensors(pkg):
    """LoRA X -> none -> LoRA Y with factors in a non-compute dtype (so converted copies exist): the converted
    factors must be Y's, also when Y's tensors sit where X's were.  The cache entry holds the source tensors and is
    matched by identity, and the hook drops it whenever it replaces them."""
    o = pkg.ops
    mod = types.SimpleNamespace(lora_A=None, lora_B=None, lora_alpha=None, _lora_cache=None)
    cpu = torch.device("cpu")
    xa, xb = torch.full((4, 16), 1.0, dtype=torch.float16), torch.full((8, 4), 2.0, dtype=torch.float16)
    mod.lora_A, mod.lora_B = xa, xb
    a1, b1 = o._prepare_lora(mod, cpu, torch.bfloat16)
    assert a1.dtype == torch.bfloat16 and a1.shape == (8, 16) and b1.shape == (8, 8)      # rank padded to 8
    assert o._prepare_lora(mod, cpu, torch.bfloat16)[0] is a1                              # cached while unchanged
    mod.lora_A = mod.lora_B = None
    ya, yb = torch.full((4, 16), 3.0, dtype=torch.float16), torch.full((8, 4), 4.0, dtype=torch.float16)
    mod.lora_A, mod.lora_B = ya, yb
    # the worst case: an id()-keyed cache entry that happens to match the new tensors' addresses
    mod._lora_cache = ((cpu, torch.bfloat16, None), a1, b1, xa, xb)
    a2, b2 = o._prepare_lora(mod, cpu, torch.bfloat16)
    assert float(a2[0, 0]) == 3.0 and float(b2[0, 0]) == 4.0
    # in-place edits of the same tensors keep the entry (the reference re-reads the tensors each call; the hook
    # always assigns new ones, int8_quant.py:476-496)
    hook = o.DynamicLoRAHook()
    layer = nn.Linear(16, 8)
    layer.lora_A, layer.lora_B, layer.lora_alpha, layer._lora_cache = xa, xb, None, ("stale",)
    model = nn.Sequential(layer)
    hook.apply_composition(model, [])
    assert layer.lora_A is None and layer._lora_cache is None


def test_weight_scale_length_is_checked_on_the_host(pkg):
    F = pkg.functional
    cpu = torch.device("cpu")
    ws, mode = F._wscale_arg(torch.ones(7, 1), cpu, 7)
    assert mode == pkg._native.WSCALE_CHANNEL and ws.numel() == 7 and ws.is_contiguous()
    assert F._wscale_arg(0.5, cpu, 7)[1] == pkg._native.WSCALE_TENSOR
    assert F._wscale_arg(torch.tensor(0.5), cpu, 7)[1] == pkg._native.WSCALE_TENSOR
    for bad in (torch.ones(6), torch.ones(7, 2), torch.ones(14)):
        with pytest.raises(ValueError, match="weight scale"):
            F._wscale_arg(bad, cpu, 7)
