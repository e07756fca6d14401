"""Drop-in surface: same names, same parameters and the same exception classes as
the reference's public API (chord_kernels/__init__.py:6-21, ops.py:8-90,
operator/api.py:300-315, operator/packing.py:26-60).  No GPU needed."""

import dataclasses
import inspect

import pytest
import torch


def test_public_names():
    import chord_b200
    import chord_kernels

    expected = ["contiguous", "indexed", "indexed_block_m", "masked", "pack_w4a16"]
    assert chord_kernels.__all__ == expected
    assert chord_b200.__all__ == expected
    for name in expected:
        assert getattr(chord_kernels, name) is getattr(chord_b200, name)
    with pytest.raises(AttributeError):
        chord_kernels.no_such_operator


def _params(fn):
    return [(p.name, p.kind, p.default) for p in inspect.signature(fn).parameters.values()]


def test_signatures_match_the_reference():
    import chord_b200

    P, K = inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect.Parameter.KEYWORD_ONLY
    E = inspect.Parameter.empty
    assert _params(chord_b200.indexed) == [
        ("activation", P, E), ("weight", P, E), ("sorted_ids", P, E), ("expert_ids", P, E),
        ("num_tokens_padded", P, E), ("top_k", P, E), ("locks", K, None), ("outputs", K, None),
        ("block_m", K, None), ("validate_routing", K, False)]
    assert _params(chord_b200.masked) == [
        ("activation", P, E), ("weight", P, E), ("masked_m", P, E), ("expected_m", P, E),
        ("outputs", K, None), ("enable_pdl", K, False)]
    assert _params(chord_b200.contiguous) == [
        ("activation", P, E), ("weight", P, E), ("m_indices", P, E), ("outputs", K, None),
        ("enable_pdl", K, False)]
    assert _params(chord_b200.indexed_block_m) == [
        ("weight", P, E), ("num_tokens", P, E), ("top_k", P, E), ("device", K, None),
        ("total_experts", K, None)]   # the last one is an extension (expert parallelism)
    assert _params(chord_b200.pack_w4a16) == [
        ("weight_uint4", P, E), ("weight_scale", P, E), ("packed", K, False)]
    # the schedule is not a public knob of `indexed`
    for hidden in ("config", "layout", "swap_ab"):
        assert hidden not in inspect.signature(chord_b200.indexed).parameters


def test_prepared_weight_shape():
    from chord_b200.packing import PreparedWeight

    assert [f.name for f in dataclasses.fields(PreparedWeight)] == \
        ["packed", "scale", "n", "k", "num_experts"]
    w = PreparedWeight(torch.zeros(1), torch.ones(1), 128, 64, 1)
    packed, scale = w
    assert packed is w.packed and scale is w.scale and w.tensors == (w.packed, w.scale)
    with pytest.raises(dataclasses.FrozenInstanceError):
        w.n = 3


def test_indexed_block_m_contract(native_lib):
    from chord_b200 import indexed_block_m
    from chord_b200.packing import PreparedWeight

    w = PreparedWeight(torch.zeros(1), torch.zeros(1), 4096, 7168, 48)
    for tokens in (1, 20, 50, 256, 4096):
        bm = indexed_block_m(w, tokens, 8)
        assert isinstance(bm, int) and bm % 8 == 0
    with pytest.raises(TypeError):
        indexed_block_m("not a weight", 4, 8)
    # expert parallelism: 48 of 384 experts live here, so 256 tokens x top-8 bring about
    # five rows per local expert, not forty
    assert indexed_block_m(w, 256, 8, total_experts=384) == indexed_block_m(w, 32, 8)
    assert indexed_block_m(w, 256, 8, total_experts=384) < indexed_block_m(w, 256, 8)
    assert indexed_block_m(w, 256, 8, total_experts=48) == indexed_block_m(w, 256, 8)
    with pytest.raises(ValueError):
        indexed_block_m(w, 256, 8, total_experts=8)


def test_argument_errors_before_any_gpu_work():
    import chord_b200

    cpu = torch.zeros((2, 128, 64), dtype=torch.int32)
    scale = torch.zeros((2, 128, 2), dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        chord_b200.pack_w4a16(cpu, scale, packed=1)
    with pytest.raises(TypeError):
        chord_b200.pack_w4a16([1, 2], scale)
    with pytest.raises(TypeError):
        chord_b200.pack_w4a16(cpu.to(torch.int64), scale)
    with pytest.raises(ValueError):
        chord_b200.pack_w4a16(cpu[0], scale)
    with pytest.raises(ValueError):                 # not a CUDA tensor
        chord_b200.pack_w4a16(cpu, scale)
    with pytest.raises(TypeError):
        chord_b200.indexed(torch.zeros((4, 64)), None, None, None, None, 2)
    with pytest.raises(ValueError):                 # BF16 but not on a GPU
        chord_b200.indexed(torch.zeros((4, 64), dtype=torch.bfloat16), None, None, None, None, 2)
    with pytest.raises(TypeError):
        chord_b200.masked(torch.zeros((4, 64), dtype=torch.bfloat16), "w", None, 8)
    with pytest.raises(TypeError):
        chord_b200.contiguous(torch.zeros((128, 64), dtype=torch.bfloat16), "w", None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from chord_b200 import _lib

    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setenv("CHORD_B200_LIB", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()
