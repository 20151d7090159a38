"""Merged q/k/v and gate/up projections against the separate ones, on the GPU.

The reference's gate (tests/test_merged_projections.py:42-56): for rows 1 ... 4099 the three / two
column views of the merged GEMM equal the separate projections bit for bit, and the original modules
(now views of the stacked storage) still compute the same thing.  Bit equality between GEMMs of different
N needs the single increasing-K summation order, i.e. ``set_batch_invariant(True)``; with the library free
to cut K per shape the two agree to fp32 summation order (checked separately with a bound).
"""

from __future__ import annotations

import types

import pytest
import torch

from mini_inference_engine_b200.engine.kernels import merged_projections as mp
from mini_inference_engine_b200.engine.kernels import sm89_fp8
from oracle import hot_path

pytestmark = pytest.mark.gpu

HIDDEN = 2560


class Fp8Piece(torch.nn.Module):
    """What Transformers' ``FP8Linear`` is to this path: e4m3 weight, block scales, forward = fp8_linear."""

    def __init__(self, n: int, k: int, seed: int, device) -> None:
        super().__init__()
        generator = torch.Generator().manual_seed(seed)
        w8, scales = hot_path.quantize_weight(torch.randn(n, k, generator=generator) * 0.02)
        self.weight = torch.nn.Parameter(w8.to(device), requires_grad=False)
        self.register_buffer("weight_scale_inv", scales.to(device))
        self.block_size = (128, 128)
        self.bias = None
        self.activation_scale = None

    def forward(self, x):
        return sm89_fp8.sm89_fp8_linear(x, self.weight, self.weight_scale_inv, block_size=list(self.block_size))


def _owner(names, widths, device):
    return types.SimpleNamespace(**{name: Fp8Piece(n, HIDDEN, 10 + i, device)
                                    for i, (name, n) in enumerate(zip(names, widths))})


CASES = ((mp.QKV, (4096, 1024, 1024), mp.project_qkv, "_minillm_qkv"),
         (mp.GATE_UP, (9728, 9728), mp.project_gate_up, "_minillm_gate_up"))


@pytest.fixture()
def batch_invariant():
    previous = sm89_fp8.set_batch_invariant(True)
    yield
    sm89_fp8.set_batch_invariant(previous)


@pytest.mark.parametrize("rows", [1, 8, 64, 255, 256, 2048, 4099])
def test_merged_equals_separate_bitwise(rows, device, batch_invariant, status_clean):
    x = torch.randn(rows, HIDDEN, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16).to(device)
    for names, widths, project, slot in CASES:
        owner = _owner(names, widths, device)
        separate = project(owner, x)
        merged = mp._stack(owner, names)
        assert merged is not None and merged.splits == widths
        owner.__dict__[slot] = merged
        # The pieces now view the stacked storage and still compute the same bits.
        assert getattr(owner, names[0]).weight.data_ptr() == merged.weight.data_ptr()
        together = project(owner, x)
        assert len(together) == len(names)
        for a, b in zip(separate, together):
            assert b.shape == a.shape and b.data_ptr() != a.data_ptr()
            assert torch.equal(a, b)
        for name, expected in zip(names, separate):
            assert torch.equal(getattr(owner, name)(x), expected)
        # Column views of ONE output.
        assert together[1].data_ptr() == together[0].data_ptr() + widths[0] * 2


@pytest.mark.parametrize("rows", [1, 64, 256])
def test_merged_close_to_separate_with_library_chosen_splits(rows, device, status_clean):
    x = torch.randn(rows, HIDDEN, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16).to(device)
    for names, widths, project, slot in CASES:
        owner = _owner(names, widths, device)
        separate = project(owner, x)
        owner.__dict__[slot] = mp._stack(owner, names)
        for a, b in zip(separate, project(owner, x)):
            # Same operands, same per-block products; only the fp32 order of adding K blocks may differ.
            bound = a.float().abs().max().item() * 2.0 ** -7
            assert (a.float() - b.float()).abs().max().item() <= bound


def test_unmergeable_pieces_are_left_alone(device):
    owner = _owner(mp.QKV, (256, 128, 128), device)
    owner.k_proj.bias = torch.nn.Parameter(torch.zeros(128, device=device))
    before = owner.q_proj.weight.data_ptr()
    assert mp._stack(owner, mp.QKV) is None
    assert owner.q_proj.weight.data_ptr() == before
    owner = _owner(mp.QKV, (256, 128, 128), device)
    owner.v_proj.weight = torch.nn.Parameter(owner.v_proj.weight[:64], requires_grad=False)  # half a scale block
    assert mp._stack(owner, mp.QKV) is None


def test_install_on_a_model_of_fp8_pieces(device):
    """``install_merged_projections`` walks a Transformers Qwen3 model; FP8 pieces stand in for FP8Linear."""

    from transformers import Qwen3Config, Qwen3ForCausalLM

    model = Qwen3ForCausalLM(Qwen3Config(
        vocab_size=64, hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
        num_key_value_heads=1, head_dim=128, max_position_embeddings=64)).to(device).to(torch.bfloat16).eval()
    assert mp.install_merged_projections(model) == 0 and mp.merged_linears(model) == []  # bf16 linears: untouched
    for layer in model.model.layers:
        attention, mlp = layer.self_attn, layer.mlp
        for name, n in (("q_proj", 256), ("k_proj", 128), ("v_proj", 128)):
            setattr(attention, name, Fp8Piece(n, 256, 1, device))
        for name in ("gate_proj", "up_proj"):
            setattr(mlp, name, Fp8Piece(256, 256, 2, device))
    assert mp.install_merged_projections(model) == 4
    assert mp.install_merged_projections(model) == 0  # idempotent
    stacks = mp.merged_linears(model)
    assert [s.splits for s in stacks] == [(256, 128, 128), (256, 256)] * 2
    x = torch.randn(3, 256, device=device).to(torch.bfloat16)
    q, k, v = mp.project_qkv(model.model.layers[0].self_attn, x)
    assert (q.shape, k.shape, v.shape) == ((3, 256), (3, 128), (3, 128)) and q.stride(0) == 512
    mp.uninstall_merged_projections(model)
    assert mp.merged_linears(model) == []
    assert mp.project_qkv(model.model.layers[0].self_attn, x)[0].stride(0) == 256
