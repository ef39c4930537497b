"""Algebraic identities the CUDA path relies on, checked on the CPU oracle (no GPU): each one is the reason a
re-formulated computation may replace the reference's literal one."""
import torch

from oracle import pom_oracle as O


def _params(D, K, E, heads=1, seed=0):
    p = O.init_params(D, K, E, heads, seed=seed, coeff_scale=0.1)
    g = torch.Generator().manual_seed(seed + 50)
    p["se_bias"] = torch.randn(p["se_bias"].shape, generator=g) * 0.3
    return {k: v.double() for k, v in p.items()}


def test_block_causal_mask_equals_one_state_forward_call_per_frame():
    """BlockCausal(L): per-frame means followed by a running mean over frames."""
    B, F, L, D, K, E = 2, 5, 12, 16, 3, 2
    model = O.OraclePoM(_params(D, K, E), K, E)
    x = torch.randn(B, F * L, D, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    want = model.forward(x, mask=O.block_causal_mask(F * L, L, B, dtype=torch.float64))
    state, outs = None, []
    for f in range(F):
        y, state = model.state_forward(x[:, f * L:(f + 1) * L], None, state)
        outs.append(y)
    assert torch.allclose(torch.cat(outs, 1), want, rtol=1e-10, atol=1e-12)


def test_grouped_projection_equals_dense_block_diagonal_weight():
    """n_groups > 1 runs as one dense GEMM on the block-diagonal weight."""
    B, N, D, K, E, g = 2, 9, 16, 2, 2, 4
    P = D * E
    gen = torch.Generator().manual_seed(2)
    w_po = torch.randn(P, D // g, 1, generator=gen, dtype=torch.float64)
    grouped = {"po_proj.weight": w_po, "se_proj.weight": torch.randn(P, D, generator=gen, dtype=torch.float64),
               "se_proj.bias": torch.randn(P, generator=gen, dtype=torch.float64),
               "po_coeff": torch.randn(P, K, generator=gen, dtype=torch.float64) * 0.1,
               "ag_proj.weight": torch.randn(D, P, generator=gen, dtype=torch.float64)}
    dense_w = torch.block_diag(*w_po.squeeze(-1).view(g, P // g, D // g).unbind(0))
    dense = {"qc_proj.weight": torch.cat([dense_w, grouped["se_proj.weight"]], 0), "se_bias": grouped["se_proj.bias"],
             "po_coeff": grouped["po_coeff"], "ag_proj.weight": grouped["ag_proj.weight"]}
    x = torch.randn(B, N, D, generator=gen, dtype=torch.float64)
    for mask in (None, "causal"):
        a = O.OraclePoM(grouped, K, E).forward(x, mask=mask)
        b = O.OraclePoM(dense, K, E).forward(x, mask=mask)
        assert torch.allclose(a, b, rtol=1e-10, atol=1e-12)


def test_multi_head_gate_collapses_to_a_heads_by_dim_matrix_per_sample():
    """y[b] = s[b] (T x heads) · Mb[b] (heads x D) with Mb[b, h, :] = sum over the channels p of head h of
    H[b, p] * Wo[:, p], when the aggregate H is per sample."""
    B, N, D, K, E, heads = 2, 11, 16, 2, 2, 4
    P = D * E
    params = _params(D, K, E, heads, seed=3)
    model = O.OraclePoM(params, K, E, heads)
    x = torch.randn(B, N, D, generator=torch.Generator().manual_seed(4), dtype=torch.float64)
    want = model.forward(x)
    hp, s = model.project(x, x)                              # s: (B, N, heads)
    H = O.aggregate(O.poly_features(hp, params["po_coeff"]), None)   # (B, 1, P)
    Mb = torch.einsum("bhj,dhj->bhd", H.view(B, heads, P // heads), params["ag_proj.weight"].view(D, heads, P // heads))
    got = torch.einsum("bth,bhd->btd", s, Mb)
    assert torch.allclose(got, want, rtol=1e-10, atol=1e-12)


def test_aggregate_of_token_shards_is_the_sum_of_shard_partials():
    """Token sharding: the (B, P) aggregate is a sum over ranks of local sums, the causal prefix needs only the
    totals of the ranks before."""
    B, N, D, K, E, W = 2, 24, 16, 2, 2, 3
    params = _params(D, K, E, seed=5)
    model = O.OraclePoM(params, K, E)
    x = torch.randn(B, N, D, generator=torch.Generator().manual_seed(6), dtype=torch.float64)
    full = model.forward(x, mask="causal")
    n = N // W
    feats = [O.poly_features(model.project(x[:, r * n:(r + 1) * n], x[:, r * n:(r + 1) * n])[0], params["po_coeff"])
             for r in range(W)]
    for r in range(W):
        carry = sum((f.sum(1) for f in feats[:r]), torch.zeros(B, D * E, dtype=torch.float64))
        y = model.forward(x[:, r * n:(r + 1) * n], mask="causal", token_offset=r * n, carry=carry)
        assert torch.allclose(y, full[:, r * n:(r + 1) * n], rtol=1e-10, atol=1e-12)
