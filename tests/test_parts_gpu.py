"""Each part of a layer alone against the plain implementation's function for it."""
import pytest
import torch

from tests import harness
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["float32", "bfloat16"]


def close(actual, expected, dtype, scale=1.0):
    if dtype == torch.float32:
        torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), atol=1e-5 * scale, rtol=1e-5)
    else:
        torch.testing.assert_close(actual.float().cpu(), expected.float().cpu(), atol=1.6e-2 * scale, rtol=1.6e-2)


def fill(part, seed, dtype):
    """Random parameters (rounded to bfloat16 so that both dtypes see the same numbers); returns name -> CPU float32."""
    from qwen_inference_lab_b200.weights.random_init import draw
    values = {}
    for name, param in part.all_named_params().items():
        value = draw(param, seed, name, dtype=torch.bfloat16)
        if param.init == "zeros":
            value = (torch.randn(param.shape, generator=torch.Generator().manual_seed(seed)) * 0.1).to(torch.bfloat16)
        values[name] = value.float()
        param.data = value.to(dtype).cuda()
    part.finalize(torch.device("cuda"), dtype)
    return values


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("bias", [False, True])
def test_linear(dtype, bias):
    from qwen_inference_lab_b200.parts import Linear, StackedLinear
    torch.manual_seed(0)
    x = torch.randn(9, 72).to(dtype)
    residual = torch.randn(9, 40).to(dtype)
    part = Linear(72, 40, name="p", bias=bias)
    w = fill(part, 1, dtype)
    expected = plain.linear(x.float(), w["p.weight"], w.get("p.bias"))
    close(part.forward(None, x.cuda()), expected, dtype, scale=0.3)
    close(part.forward(None, x.cuda(), residual=residual.cuda().clone()), expected + residual.float(), dtype, scale=3)
    logits = part.forward(None, x.cuda(), out_float32=True)
    assert logits.dtype == torch.float32
    close(logits, expected, dtype, scale=0.3)
    stacked = StackedLinear(72, [("a", 24), ("b", 8), ("c", 8)], bias=bias)
    w = fill(stacked, 2, dtype)
    expected = torch.cat([plain.linear(x.float(), w[f"{n}.weight"], w.get(f"{n}.bias")) for n in "abc"], dim=1)
    close(stacked.forward(None, x.cuda()), expected, dtype, scale=0.3)


def test_linear_with_a_float32_weight_under_bfloat16_activations():
    from qwen_inference_lab_b200.parts import Linear
    torch.manual_seed(1)
    part = Linear(50, 30, name="p")
    weight = torch.randn(30, 50) * 0.1 + 1e-4
    part.weight.data = weight.cuda()                       # stays 32-bit
    x = torch.randn(4, 50).to(torch.bfloat16)
    out = part.forward(None, x.cuda())
    assert out.dtype == torch.bfloat16
    close(out, x.float() @ weight.t(), torch.bfloat16)
    exact = part.forward(None, x.cuda(), out_float32=True)
    torch.testing.assert_close(exact.cpu(), x.float() @ weight.t(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_rmsnorm_part(dtype):
    from qwen_inference_lab_b200.parts import RMSNorm
    part = RMSNorm(200, 1e-5, name="n")
    w = fill(part, 3, dtype)
    x = (torch.randn(6, 200) * 2).to(dtype)
    close(part.forward(None, x.cuda()), plain.rms_norm(x, w["n.weight"].to(dtype), 1e-5), dtype, scale=2)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_rotary_table_is_the_references_coefficients(dtype):
    """cos and sin of float32 angles, rounded to the activation dtype, bit for bit
    (tests/qil/test_bf16.py:47-65 pins the same property of the reference)."""
    from qwen_inference_lab_b200.parts import RotaryEmbedding
    part = RotaryEmbedding(128, 1000000.0, 2048)
    part.finalize(torch.device("cuda"), dtype)
    angles = plain.rotary_angles(torch.arange(2048), 128, 1000000.0)
    table = part.table.cpu()
    assert table.dtype == torch.float32 and table.shape == (2048, 128)
    assert torch.equal(table[:, :64], angles.cos().to(dtype).float())
    assert torch.equal(table[:, 64:], angles.sin().to(dtype).float())
    with pytest.raises(ValueError):
        RotaryEmbedding(7, 10000.0, 16)


ATTENTION_SHAPES = [dict(hidden=64, n_q=4, n_kv=2, d=16, bias=False, eps=1e-6, theta=10000.0),
                    dict(hidden=96, n_q=6, n_kv=2, d=32, bias=True, eps=1e-5, theta=1e6),
                    dict(hidden=80, n_q=5, n_kv=1, d=48, bias=True, eps=3e-6, theta=50000.0)]


def attention_reference(x, w, shape, angles):
    cfg = dict(num_attention_heads=shape["n_q"], num_key_value_heads=shape["n_kv"], head_dim=shape["d"],
               rms_norm_eps=shape["eps"])
    return plain.attention_block(x, w, "", cfg, angles)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("shape", ATTENTION_SHAPES, ids=["d16", "d32", "d48"])
def test_attention_part_whole_and_cut(dtype, shape):
    from qwen_inference_lab_b200.parts import GroupedQueryAttention, RotaryEmbedding
    names = {k: f"self_attn.{k}_proj" for k in "qkvo"} | {"q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm"}
    part = GroupedQueryAttention(shape["hidden"], shape["n_q"], shape["n_kv"], shape["d"], names=names,
                                 bias=shape["bias"], qk_norm_eps=shape["eps"],
                                 position=RotaryEmbedding(shape["d"], shape["theta"], 512))
    w = fill(part, 4, dtype)
    torch.manual_seed(5)
    inputs = {"a": torch.randn(150, shape["hidden"]).to(torch.bfloat16).float(),
              "b": torch.randn(37, shape["hidden"]).to(torch.bfloat16).float()}
    expected = {rid: attention_reference(x, w, shape, plain.rotary_angles(torch.arange(len(x)), shape["d"], shape["theta"]))
                for rid, x in inputs.items()}
    body = lambda ctx, x, view: part.forward(ctx, x, view)
    whole = harness.run_part(part, shape["hidden"], dtype, body, inputs, {"a": [150], "b": [37]})
    cut = harness.run_part(part, shape["hidden"], dtype, body, inputs,
                           {"a": [70, 1, 1, 2, 65, 1, 10], "b": [1, 1, 30, 5]})
    for rid in inputs:
        close(whole[rid], expected[rid], dtype, scale=0.3)
        close(cut[rid], expected[rid], dtype, scale=0.3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_gated_mlp_part(dtype):
    from qwen_inference_lab_b200.parts import GatedMLP
    part = GatedMLP(96, 200, names={k: f"mlp.{k}_proj" for k in ("gate", "up", "down")})
    w = fill(part, 6, dtype)
    x = torch.randn(11, 96).to(torch.bfloat16).float()
    residual = torch.randn(11, 96).to(torch.bfloat16).float()
    expected = plain.gated_mlp(x, w, "")
    close(part.forward(None, x.to(dtype).cuda()), expected, dtype, scale=0.1)
    close(part.forward(None, x.to(dtype).cuda(), residual=residual.to(dtype).cuda()), expected + residual, dtype, scale=3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_block_part(dtype):
    from qwen_inference_lab_b200.parts import GatedMLP, GroupedQueryAttention, PreNormBlock, RMSNorm, RotaryEmbedding
    shape = ATTENTION_SHAPES[1]
    prefix = "model.layers.0."
    names = {k: prefix + f"self_attn.{k}_proj" for k in "qkvo"} | {"q_norm": prefix + "self_attn.q_norm",
                                                                   "k_norm": prefix + "self_attn.k_norm"}
    block = PreNormBlock(
        RMSNorm(shape["hidden"], shape["eps"], name=prefix + "input_layernorm"),
        GroupedQueryAttention(shape["hidden"], shape["n_q"], shape["n_kv"], shape["d"], names=names, bias=shape["bias"],
                              qk_norm_eps=shape["eps"], position=RotaryEmbedding(shape["d"], shape["theta"], 256)),
        RMSNorm(shape["hidden"], shape["eps"], name=prefix + "post_attention_layernorm"),
        GatedMLP(shape["hidden"], 136, names={k: prefix + f"mlp.{k}_proj" for k in ("gate", "up", "down")}))
    w = fill(block, 7, dtype)
    torch.manual_seed(8)
    inputs = {"a": torch.randn(45, shape["hidden"]).to(torch.bfloat16).float()}
    cfg = dict(num_attention_heads=shape["n_q"], num_key_value_heads=shape["n_kv"], head_dim=shape["d"],
               rms_norm_eps=shape["eps"])
    expected = plain.decoder_block(inputs["a"], w, prefix, cfg, plain.rotary_angles(torch.arange(45), shape["d"], shape["theta"]))
    body = lambda ctx, x, view: block.forward(ctx, x, view)
    out = harness.run_part(block, shape["hidden"], dtype, body, inputs, {"a": [20, 2, 23]})
    close(out["a"], expected, dtype, scale=3)
