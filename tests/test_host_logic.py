"""Host-side arithmetic of the C ABI that needs no GPU: buffer layouts, workspace sizes, argument checks."""
import ctypes as C

import pytest

from pom_b200 import _abi, _build


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _abi.lib()


def test_peer_layout_offsets(lib):
    lay = (C.c_ulonglong * 3)()
    assert lib.pom_peer_layout(8, 4096, 1024, lay) == 0
    assert lay[0] == 65536                                   # header
    assert lay[1] == lay[0] + 2 * 8 * 4096 * 4               # two epochs x eight writers x slot
    assert lay[2] == lay[1] + 1024 * (4 + 2 + 2)             # fp32 accumulators + bf16 staging and result images
    assert lib.pom_peer_layout(17, 4096, 0, lay) < 0         # more ranks than the header has flags for
    assert lib.pom_peer_layout(2, 4095, 0, lay) < 0          # slots are multiples of 4 floats (16-byte accesses)


def test_layer_workspace_covers_both_passes(lib):
    a = _abi.LayerArgs()
    a.B, a.T, a.N, a.D, a.P, a.K = 32, 1024, 1024, 1152, 2304, 2
    a.self_mixing, a.frames = 1, 1
    n = int(lib.pom_layer_workspace_bytes(C.byref(a)))
    bp = 32 * 2304 * 4
    fwd = 8 * bp + bp                       # per-tile sums of 8 m-tiles + one (B, P) vector
    bwd = 2 * 8 * bp + 16 * bp * 2 + 2 * bp  # two partial sets, coefficient partials (16 chunks x K), two vectors
    assert n >= max(fwd, bwd) and n < 2 * max(fwd, bwd)
    a.N = 0
    assert int(lib.pom_layer_workspace_bytes(C.byref(a))) == 0


def test_layer_entry_points_validate_before_touching_the_gpu(lib):
    a = _abi.LayerArgs()
    assert lib.pom_layer_fwd(C.byref(a), None, None) == -8      # null pointers
    a.B, a.T, a.N, a.D, a.P, a.K = 2, 16, 16, 60, 120, 2         # D not a multiple of 8
    a.self_mixing, a.frames = 1, 1
    dummy = C.c_void_p(256)
    for f in ("xq", "w_qc", "w_ag", "se_bias", "coeff", "H", "workspace"):
        setattr(a, f, dummy)
    a.workspace_bytes = 1 << 30
    assert lib.pom_layer_fwd(C.byref(a), None, None) == -3      # alignment
    a.D, a.P, a.K = 64, 128, 17
    assert lib.pom_layer_fwd(C.byref(a), None, None) == -5      # degree above 16
    a.K, a.frames = 2, 3                                         # B not a multiple of frames
    assert lib.pom_layer_fwd(C.byref(a), None, None) == -1
    a.frames, a.workspace_bytes = 1, 16
    assert lib.pom_layer_fwd(C.byref(a), None, None) == -9      # workspace too small


def test_gemm_entry_point_validates_before_touching_the_gpu(lib):
    g = _abi.GemmArgs()
    assert lib.pom_gemm_bf16(C.byref(g), None, None) == -8       # null operands
    g.A = g.Bm = g.C = 0x1000
    assert lib.pom_gemm_bf16(C.byref(g), None, None) == -1       # empty problem
    g.M, g.N, g.K, g.batches = 128, 128, 64, 1
    g.lda, g.ldb, g.ldc = 60, 64, 128
    assert lib.pom_gemm_bf16(C.byref(g), None, None) == -2       # row stride not a multiple of 8 elements
    g.lda, g.ldc = 32, 128
    assert lib.pom_gemm_bf16(C.byref(g), None, None) == -2       # row stride shorter than a row
    lib.pom_strerror.restype = C.c_char_p
    texts = {code: lib.pom_strerror(code) for code in range(0, -10, -1)}
    assert all(t for t in texts.values()) and len(set(texts.values())) == 10  # one message per code


def test_backward_partial_slot_count_never_exceeds_the_chunk_capacity(lib):
    a = _abi.AggBwdArgs()
    for B, N, P in ((32, 1024, 2304), (1, 65536, 2304), (64, 2048, 2048), (3, 70, 96), (2, 320, 256), (2, 24, 32)):
        a.B, a.N, a.P, a.K = B, N, P, 2
        a.dtype, a.causal = 0, 0
        a.ldx = a.ld_dx = P
        a.x = a.dx = C.c_void_p(512)
        slots = lib.pom_poly_agg_bwd_slots(C.byref(a))
        assert 0 < slots <= B * lib.pom_agg_chunks(N)
        # the fused token-causal form walks 32-token tiles: its runs must fit the same capacity
        a.causal, a.dout, a.partial, a.ld_dout = 3, C.c_void_p(512), C.c_void_p(512), P
        slots = lib.pom_poly_agg_bwd_slots(C.byref(a))
        assert 0 < slots <= B * lib.pom_agg_chunks(N), (B, N, P, slots)
        a.causal, a.dout, a.partial = 0, None, None


def _module_for(cfg):
    from pom_b200 import PoM, PoMRoPE

    r = cfg.get("rope")
    args = (cfg["dim"], cfg["degree"], cfg["expand"], cfg.get("groups", 1), cfg["heads"])
    if r is None:
        return PoM(*args, bias=cfg.get("bias", False))
    return PoMRoPE(*args, bias=cfg.get("bias", False), rope_2d=r["two_d"], max_seq_len=r.get("max_seq_len", 4096), max_h=r.get("max_h", 64),
                   max_w=r.get("max_w", 64))


@pytest.mark.parametrize("name", ["pom_none", "pom_heads4_none", "pom_groups2_none", "pom_groups2_heads4_none",
                                  "pom_groups2_bias_none",
                                  "rope1d_none", "rope2d_none", "rope2d_heads4_none"])
def test_reference_state_dicts_load_strictly_and_round_trip(golden, name):
    """Checkpoints interchange with the reference: same parameter and buffer names and shapes, and the rotary
    tables the module builds equal the reference's buffers."""
    import torch

    case = golden[name]
    mod = _module_for(case["cfg"])
    own = mod.state_dict()
    assert sorted(own.keys()) == sorted(case["params"].keys())
    for k, v in case["params"].items():
        assert own[k].shape == v.shape, k
        if "cos" in k or "sin" in k:  # tables are deterministic functions of the constructor arguments
            assert torch.allclose(own[k], v, atol=1e-6, rtol=0), k
    mod.load_state_dict(case["params"], strict=True)
    back = mod.state_dict()
    for k, v in case["params"].items():
        assert torch.equal(back[k], v), k


def test_shape_errors_are_raised_before_any_device_work():
    """mask="causal" pairs query token m with the prefix aggregate of context token m: different lengths are an
    error (the reference asserts the same in its selection step), as are mismatched batch or feature sizes."""
    import torch

    from pom_b200 import PoM

    mod = PoM(16, 2, 2)
    xq, xc = torch.randn(2, 6, 16), torch.randn(2, 9, 16)
    with pytest.raises(ValueError, match="causal"):
        mod(xq, xc, mask="causal")
    with pytest.raises(ValueError, match="batch"):
        mod(xq, torch.randn(3, 6, 16))
    with pytest.raises(ValueError, match="feature"):
        mod(xq, torch.randn(2, 6, 8))


def test_grouped_projection_is_assembled_once_per_parameter_version():
    """Without autograd the block-diagonal form of the grouped projection is reused until a parameter changes;
    with autograd it stays part of the graph of every call (reference pom/pom.py:180-183, 203-205)."""
    import torch
    from pom_b200 import PoM

    torch.manual_seed(0)
    m = PoM(16, 2, 2, n_groups=4)
    with torch.no_grad():
        w1, _ = m._weights()
        w2, _ = m._weights()
        assert w1 is w2
        blocks = m.po_proj.weight.squeeze(-1).view(4, 8, 4)
        assert torch.equal(w1[:8, :4], blocks[0]) and torch.equal(w1[24:32, 12:16], blocks[3])
        assert float(w1[:8, 4:].abs().max()) == 0.0
        assert torch.equal(w1[32:], m.se_proj.weight)
        m.po_proj.weight.mul_(2.0)  # in-place update: new version, new matrix
        w3, _ = m._weights()
        assert w3 is not w1 and torch.equal(w3[:8, :4], blocks[0])
    w4, _ = m._weights()  # autograd on: rebuilt and differentiable
    assert w4.requires_grad and w4 is not w3
    w4.sum().backward()
    assert m.po_proj.weight.grad is not None and float(m.po_proj.weight.grad.min()) == 1.0


def test_operator_module_carries_the_reference_names():
    """Every operator function the reference's tests and benchmarks import has a namesake in pom_b200.operators
    (pom/pom_triton.py:383, pom_triton_causal.py:400, pom_triton_masked.py:402, pom_triton_rope.py:985, 1020,
    pom/pom.py:27, pom/pom_rope.py:152, 183), and the CPU is refused rather than served by a fallback."""
    import torch

    from pom_b200 import operators, pom_rope

    for name in ("poly_agg_mean_triton", "poly_agg_causal_triton", "poly_agg_masked_triton",
                 "poly_agg_rope_mean_triton", "poly_agg_rope_causal_triton", "pom_activation", "apply_rope_1d",
                 "apply_rope_2d", "poly_features"):
        assert callable(getattr(operators, name)), name
    assert pom_rope.apply_rope_1d is operators.apply_rope_1d and pom_rope.apply_rope_2d is operators.apply_rope_2d
    # the import lines of the reference's scripts, with the package name changed
    from pom_b200 import PoM, PoMRoPE, pom  # noqa: F401  (pom/__init__.py)
    from pom_b200.pom import polynomial_aggregation_, polynomial_selection_, pom_activation  # noqa: F401
    from pom_b200.pom import pom as pom_fn
    from pom_b200.pom_rope import precompute_freqs_1d, precompute_freqs_2d  # noqa: F401

    assert callable(pom) and pom is pom_fn and not isinstance(pom, type(operators))
    with pytest.raises(RuntimeError, match="no CPU path"):
        operators.pom_activation(torch.randn(2, 3, 8))
    with pytest.raises(RuntimeError, match="no CPU path"):
        operators.apply_rope_1d(torch.randn(1, 4, 8), torch.arange(4), torch.ones(4, 4), torch.zeros(4, 4))


def test_row_strides_ignore_dimensions_of_size_one():
    """PyTorch reports arbitrary strides for dimensions of size 1; the leading dimension handed to the library must
    not depend on them."""
    import torch

    from pom_b200.ops import _ld, _row_stride

    wide = torch.zeros(3, 1, 12)
    assert _row_stride(wide[..., :8]) == 12                    # (3, 1, 8) slice of rows that are 12 long
    assert _row_stride(torch.zeros(1, 5, 12)[..., :8]) == 12   # one sample: the token stride decides
    assert _row_stride(torch.zeros(1, 1, 12)[..., :8]) == 8    # a single row: any stride would do, the tight one
    assert _row_stride(torch.zeros(1, 12)[:, :8]) == 8
    assert _row_stride(torch.zeros(4, 12)[:, :8]) == 12
    odd = torch.zeros(3, 1, 8).as_strided((3, 1, 8), (8, 999, 1))
    assert _row_stride(odd) == 8 and _ld(odd, 1) == 8
    padded = torch.zeros(2, 1, 8)[..., :1]                      # one mask row of one element, rows padded to 8
    assert _ld(padded, 1) == 8 and _ld(torch.zeros(2, 1, 3), 1) == 8 and _ld(torch.zeros(2, 5, 16), 1) == 16
    with pytest.raises(ValueError):
        _row_stride(torch.zeros(2, 6, 8)[:, :5])               # batch and token dimensions do not collapse


def test_batch_slices_and_mask_operand():
    import torch

    from pom_b200 import functional as Fn

    sl = Fn._batch_slices(70000)
    assert [(s.start, s.stop) for s in sl] == [(0, 65535), (65535, 70000)]
    assert [(s.start, s.stop) for s in Fn._batch_slices(10, 4)] == [(0, 4), (4, 8), (8, 10)]
    assert Fn._batch_slices(5, 0)[0] == slice(0, 1)            # never an empty or endless cut
    assert Fn._cut("causal", sl[0]) == "causal" and Fn._cut(None, sl[0]) is None
    m = (torch.rand(2, 3, 37) < 0.5)
    op = Fn._mask_operand(m, "cpu", torch.bfloat16)
    assert op.shape == (2, 3, 37) and op.stride() == (3 * 40, 40, 1) and torch.equal(op.float(), m.float())
    dense = Fn._mask_operand(torch.ones(2, 3, 40), "cpu", torch.float32)
    assert dense.is_contiguous()
    assert torch.equal(Fn._inv_rows(torch.tensor([0.0, 2.0, 4.0])), torch.tensor([0.0, 0.5, 0.25]))


def test_gate_heads_are_repeated_up_to_a_multiple_of_eight_in_bf16():
    """4 heads -> 8 (two copies each), 12 -> 24, 16 stays, fp32 stays; the repeated gate weight and bias keep every
    copy next to its original, and the cache of the assembled projection follows in-place updates."""
    import torch

    from pom_b200 import PoM

    for heads, want in ((4, 2), (12, 2), (16, 1), (6, 4), (3, 8)):
        m = PoM(48, 2, 2, n_sel_heads=heads)
        assert m._head_copies() == 1 and m._heads() == heads
        m.bfloat16()
        assert m._head_copies() == want and m._heads() == heads * want
        with torch.no_grad():
            w, b = m._weights()
            assert w.shape == (96 + heads * want, 48) and b.shape == (heads * want,)
            assert torch.equal(w[96:], m.qc_proj.weight[96:].repeat_interleave(want, 0))
            if want > 1:
                assert m._weights()[0] is w                    # kept while the parameters are unchanged
                m.se_bias.add_(1.0)
                assert torch.equal(m._weights()[1], m.se_bias.repeat_interleave(want))


def test_grouped_bias_travels_as_an_input_channel():
    import torch

    from pom_b200 import PoM

    m = PoM(16, 2, 2, n_groups=2, bias=True)
    with torch.no_grad():
        m.po_proj.bias.copy_(torch.arange(32.0))
        w, _ = m._weights()
    assert w.shape == (64, 24) and torch.equal(w[:32, 16], torch.arange(32.0)) and float(w[32:, 16:].abs().sum()) == 0
    x = m._tokens(torch.zeros(2, 3, 16))
    assert x.shape == (2, 3, 24) and float(x[..., 16].min()) == 1.0 and float(x[..., 17:].abs().sum()) == 0
    assert m._out_weight().shape == (24, 32) and float(m._out_weight()[16:].detach().abs().sum()) == 0
    assert PoM(16, 2, 2, n_groups=2)._tokens(torch.zeros(1, 1, 16)).shape == (1, 1, 16)
