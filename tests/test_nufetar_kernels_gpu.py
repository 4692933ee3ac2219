"""The kernels Nufetar brought, each alone against plain torch in float64: attention with a group of heads per
CTA (score mix, runs of positions, windows, head gates, values read out of the key rows), the preparation of
queries, keys and values (both pairings of the rotation, value norm, float32 queries), the latent row's preparation,
the product per head, the token shift with its state, the recurrence, and the learned activation."""
import math

import pytest
import torch

import plain_nufetar as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
ACT = [torch.float32, torch.bfloat16]


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


def paged(rows, n_heads, width, page, dtype, n_pages, order):
    """A pool [n_pages, heads, page, width] holding ``rows [T, heads, width]`` of one request in the pages ``order``
    (the others filled with NaN: reading a page nobody was given shows)."""
    T = rows.shape[0]
    pool = torch.full((n_pages, n_heads, page, width), float("nan"), dtype=dtype, device=DEV)
    for t in range(T):
        pool[order[t // page], :, t % page, :rows.shape[2]] = rows[t].to(dtype).to(DEV)
        pool[order[t // page], :, t % page, rows.shape[2]:] = 0
    return pool


def check_tiles(ops, qd, qhs, table, kp, vp, H, dk, dv, scale, window, chunk, talk, gate, want, T):
    """The tensor-core kernel over the same request: as portions in tiles of up to 128 queries (one of them cut short,
    one empty), and as single-token rows; float32 and bfloat16 outputs."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tiles = i32([[128, T - 128, 0, 128], [0, 0, 0, 0], [0, 128, 0, 0]])
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((T, H * dv), 7.0, dtype=out_dtype, device=DEV)
        ops.attention_wide_tiles(qd, qhs, tiles, 3, 128, table, kp, vp, out, dv, H, dk, dv, scale, status,
                                 ops.current_stream(), window=window, chunk=chunk, talk=talk, gate=gate)
        assert int(status.item()) == 0
        err = float((out.double().cpu().view(T, H, dv) - want).abs().max())
        assert err < (6e-3 if out_dtype == torch.float32 else 2e-2), ("tiles", out_dtype, err)
    rows = [0, 1, 63, 64, 65, 127, 128, T - 1]
    singles = i32([[r, 1, 0, r] for r in rows] + [[5, 0, 0, 0]])
    out = torch.full((T, H * dv), 7.0, device=DEV)
    ops.attention_wide_tiles(qd, qhs, singles, len(rows) + 1, 1, table, kp, vp, out, dv, H, dk, dv, scale, status,
                             ops.current_stream(), window=window, chunk=chunk, talk=talk, gate=gate)
    assert int(status.item()) == 0
    got = out.double().cpu().view(T, H, dv)
    assert float((got[rows] - want[rows]).abs().max()) < 6e-3
    assert bool((out[5] == 7.0).all()) and bool((out[2] == 7.0).all())
    # the same rows with their keys split over several CTAs and merged
    need = ops.attention_wide_scratch(len(rows) + 1, H, dv, window, chunk, 4096)
    assert (need > 0) == (min(x for x in (window, chunk, 4096) if x) > 128)
    if need:
        scratch = torch.full((need,), float("nan"), device=DEV)
        out2 = torch.full((T, H * dv), 7.0, device=DEV)
        ops.attention_wide_tiles(qd, qhs, singles, len(rows) + 1, 1, table, kp, vp, out2, dv, H, dk, dv, scale, status,
                                 ops.current_stream(), window=window, chunk=chunk, talk=talk, gate=gate, scratch=scratch,
                                 max_len=4096)
        assert int(status.item()) == 0
        assert float((out2.double().cpu().view(T, H, dv)[rows] - want[rows]).abs().max()) < 6e-3
        assert bool((out2[5] == 7.0).all()) and bool((out2[2] == 7.0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,G,dk,dv,window,chunk,talk,gate", [
    (4, 2, 32, 16, 0, 24, True, True),
    (3, 3, 48, 40, 0, 100, True, False),
    (6, 1, 16, 24, 0, 7, True, True),
    (8, 2, 64, 64, 50, 0, False, False),
    (8, 4, 64, 64, 0, 0, True, True),          # every key visible: single rows split over several CTAs
    (2, 2, 20, 7, 33, 64, True, True),        # rows that are no multiple of 16 bytes, an odd value width
    (1, 1, 8, 8, 1, 0, True, True),
])
def test_attention_with_a_group_of_heads(act, H, G, dk, dv, window, chunk, talk, gate):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * dk + dv + window + chunk)
    T, page = 150, 16
    q = torch.randn(T, H, dk)
    k = torch.randn(T, G, dk).to(act).float()
    v = torch.randn(T, G, dv).to(act).float()
    Tm = (torch.eye(H) + 0.3 * torch.randn(H, H)) if talk else None
    gt = torch.randn(T, H).to(act).float() if gate else None
    scale = 0.6 / math.sqrt(dk) * 3
    # plain
    rep = H // G
    raw = torch.stack([q[:, h].double() @ k[:, h // rep].double().T for h in range(H)]) * scale
    mixed = torch.einsum("hg,gij->hij", Tm.double(), raw) if talk else raw
    mask = plain.visible(T, window=window or None, chunk=chunk or None)
    want = torch.stack([plain.softmax_rows(mixed[h], mask) @ v[:, h // rep].double() for h in range(H)], dim=1)
    if gate:
        want = want * torch.sigmoid(gt.double())[:, :, None]
    n_pages = (T + page - 1) // page
    order = list(reversed(range(n_pages)))
    krow, vrow = (dk + 7) // 8 * 8, (dv + 7) // 8 * 8
    kp, vp = paged(k, G, krow, page, act, n_pages + 1, order), paged(v, G, vrow, page, act, n_pages + 1, order)
    table = i32([order + [-1] * 3])
    qd = torch.zeros(T, H * krow, device=DEV)
    qd.view(T, H, krow)[:, :, :dk] = q.to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for out_dtype in {act, torch.float32}:
        out = torch.zeros(T, H * dv, dtype=out_dtype, device=DEV)
        ops.attention_wide(qd, krow, i32(list(range(T))), i32([0] * T), table, kp, vp, out, dv, H, dk, dv, scale, status,
                           ops.current_stream(), window=window, chunk=chunk, talk=Tm.to(DEV).contiguous() if talk else None,
                           gate=gt.to(act).to(DEV) if gate else None)
        assert int(status.item()) == 0
        err = float((out.double().cpu().view(T, H, dv) - want).abs().max())
        assert err < (2e-5 if out_dtype == torch.float32 else 2e-2), (out_dtype, err)
    if act == torch.bfloat16:
        assert ops.attention_wide_tc_supported(kp, vp, H, dk, dv, talk) == (dk % 8 == 0 and dv % 8 == 0)
        if ops.attention_wide_tc_supported(kp, vp, H, dk, dv, talk):
            check_tiles(ops, qd, krow, table, kp, vp, H, dk, dv, scale, window, chunk,
                        Tm.to(DEV).contiguous() if talk else None, gt.to(act).to(DEV) if gate else None, want, T)
    # a row that pads the step is skipped; a subset of rows leaves the others alone
    out = torch.full((T, H * dv), 7.0, device=DEV)
    req = [0] * T
    req[5] = -1
    ops.attention_wide(qd, krow, i32(list(range(T))), i32(req), table, kp, vp, out, dv, H, dk, dv, scale, status,
                       ops.current_stream(), window=window, chunk=chunk, talk=Tm.to(DEV).contiguous() if talk else None,
                       gate=gt.to(act).to(DEV) if gate else None, rows=i32([3, 5, 149]))
    assert float((out[3].double().cpu().view(H, dv) - want[3]).abs().max()) < 2e-5
    assert float((out[149].double().cpu().view(H, dv) - want[149]).abs().max()) < 2e-5
    assert bool((out[5] == 7.0).all()) and bool((out[4] == 7.0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,R,dr,window", [(4, 24, 8, 20), (1, 40, 16, 2), (6, 30, 6, 0), (16, 128, 32, 64)])
def test_attention_reads_values_out_of_the_key_rows(act, H, R, dr, window):
    """One pool of latent rows [c | rotated part]: keys are the whole row, values its first R columns."""
    from mlx_lm_b200 import ops
    torch.manual_seed(H + R + dr)
    T, page = 90, 16
    lat = R + dr
    row = (lat + 7) // 8 * 8
    q = torch.randn(T, H, lat)
    c = torch.randn(T, 1, lat).to(act).float()
    scale = 1.5 / math.sqrt(lat)
    mask = plain.visible(T, window=window or None)
    want = torch.stack([plain.softmax_rows(q[:, h].double() @ c[:, 0].double().T * scale, mask) @ c[:, 0, :R].double()
                        for h in range(H)], dim=1)
    n_pages = (T + page - 1) // page
    order = [(3 * i + 1) % n_pages for i in range(n_pages)] if n_pages % 3 else list(range(n_pages))
    pool = paged(c, 1, row, page, act, n_pages, order)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(T, H * R, device=DEV)
    ops.attention_wide(q.reshape(T, H * lat).to(DEV), lat, i32(list(range(T))), i32([0] * T), i32([order]), pool, pool, out,
                       R, H, lat, R, scale, status, ops.current_stream(), window=window)
    assert int(status.item()) == 0
    assert float((out.double().cpu().view(T, H, R) - want).abs().max()) < 3e-5
    if act == torch.bfloat16 and R % 8 == 0:
        assert ops.attention_wide_tc_supported(pool, pool, H, lat, R, False)
        qd = q.reshape(T, H * lat).to(DEV)
        for tiles, n, tq, rows in ((i32([[0, T, 0, 0]]), 1, 128, list(range(T))),
                                   (i32([[r, 1, 0, r] for r in (0, 1, 17, 63, 64, T - 1)]), 6, 1, [0, 1, 17, 63, 64, T - 1])):
            out = torch.zeros(T, H * R, device=DEV)
            ops.attention_wide_tiles(qd, lat, tiles, n, tq, i32([order]), pool, pool, out, R, H, lat, R, scale, status,
                                     ops.current_stream(), window=window)
            assert int(status.item()) == 0
            got = out.double().cpu().view(T, H, R)
            assert float((got[rows] - want[rows]).abs().max()) < 6e-3      # the weights are rounded to bfloat16


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("H,G,dk,dv,rot", [(4, 2, 32, 16, 16), (3, 3, 48, 40, 48), (6, 1, 16, 24, 0), (2, 2, 20, 7, 6)])
def test_queries_keys_and_values_are_prepared(act, interleaved, H, G, dk, dv, rot):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * dk + dv + rot)
    T, page, eps, base = 37, 16, 1e-5, 5000.0
    n = (H + G) * dk + G * dv
    proj = torch.randn(T, n).to(act)
    pos = torch.arange(100, 100 + T)
    turn = plain.turn_neighbours if interleaved else plain.turn_halves
    p64 = proj.double()
    q_want = turn(p64[:, :H * dk].reshape(T, H, dk), rot, base, pos)
    k_want = turn(p64[:, H * dk:(H + G) * dk].reshape(T, G, dk), rot, base, pos)
    v_want = plain.rms(p64[:, (H + G) * dk:].reshape(T, G, dv), eps)
    krow, vrow = (dk + 7) // 8 * 8, (dv + 7) // 8 * 8
    n_pages = 10
    kp = torch.full((n_pages, G, page, krow), float("nan"), dtype=act, device=DEV)
    vp = torch.full((n_pages, G, page, vrow), float("nan"), dtype=act, device=DEV)
    table = i32([[-1] * 6 + [4, 2, 9, 0]])           # positions 96.. live in logical pages 6..
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=DEV) if rot else None
    q_out = torch.full((T, H * krow), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qkv_prepare(proj.to(DEV), 0, H * dk, (H + G) * dk, H, G, dk, dv, None, None, eps, freq, i32(pos.tolist()), i32([0] * T),
                    table, kp, vp, q_out, True, status, ops.current_stream(), interleaved=interleaved, v_norm_eps=eps)
    assert int(status.item()) == 0
    tol = 1e-5 if act == torch.float32 else 3e-2
    q_got = q_out.view(T, H, krow).double().cpu()
    assert float((q_got[..., :dk] - q_want).abs().max()) < 1e-4 and bool((q_got[..., dk:] == 0).all())   # float32 queries
    for t in range(T):
        p = int(pos[t])
        pg = [4, 2, 9, 0][p // page - 6]
        assert float((kp[pg, :, p % page, :dk].double().cpu() - k_want[t]).abs().max()) < max(tol, 1e-4)
        assert float((vp[pg, :, p % page, :dv].double().cpu() - v_want[t]).abs().max()) < tol
        assert bool((kp[pg, :, p % page, dk:] == 0).all()) and bool((vp[pg, :, p % page, dv:] == 0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("H,d,dr,R", [(4, 16, 8, 24), (1, 24, 16, 40), (2, 32, 6, 30)])
def test_the_latent_row_is_prepared(act, interleaved, H, d, dr, R):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * d + dr + R)
    T, page, eps, base = 29, 16, 1e-6, 1e4
    n = H * (d + dr) + R + dr
    proj = torch.randn(T, n).to(act)
    wn = 1.0 + 0.2 * torch.randn(R)
    pos = torch.arange(3, 3 + T)
    turn = plain.turn_neighbours if interleaved else plain.turn_halves
    p64 = proj.double()
    q = p64[:, :H * (d + dr)].reshape(T, H, d + dr)
    q_rot = turn(q[..., d:], dr, base, pos)
    down = p64[:, H * (d + dr):]
    c_want = plain.rms(down[:, :R], eps) * wn.double()
    k_rot = turn(down[:, None, R:], dr, base, pos)[:, 0]
    row = (R + dr + 7) // 8 * 8
    pool = torch.full((4, 1, page, row), float("nan"), dtype=act, device=DEV)
    lat = R + dr
    q_lat = torch.full((T, H * lat), float("nan"), device=DEV)
    freq = torch.tensor([base ** (-2.0 * i / dr) for i in range(dr // 2)], dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.latent_prepare(proj.to(DEV), 0, H * (d + dr), H, d, dr, R, wn.to(DEV), eps, freq, interleaved, i32(pos.tolist()),
                       i32([0] * T), i32([[2, 0, 3]]), pool, True, q_lat, lat, status, ops.current_stream())
    assert int(status.item()) == 0
    tol = 1e-5 if act == torch.float32 else 3e-2
    assert float((q_lat.view(T, H, lat)[..., R:].double().cpu() - q_rot).abs().max()) < 1e-4
    for t in range(T):
        p = int(pos[t])
        got = pool[[2, 0, 3][p // page], 0, p % page].double().cpu()
        assert float((got[:R] - c_want[t]).abs().max()) < tol and float((got[R:lat] - k_rot[t]).abs().max()) < max(tol, 1e-4)
        assert bool((got[lat:] == 0).all())


@pytest.mark.parametrize("H,N,K,T", [(4, 24, 16, 37), (1, 40, 24, 200), (6, 64, 8, 5), (3, 70, 130, 65)])
def test_a_product_per_head(H, N, K, T):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * N + K)
    for wdt, xdt, odt in [(torch.float32, torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16, torch.float32),
                          (torch.bfloat16, torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32, torch.float32)]:
      # heads lie apart by more than their own width; the second pair: strides that allow 16-byte loads
      for xs, os_ in ((K + 3, N + 5), ((K + 7) // 8 * 8 + 8, N + 16)):
          x = torch.randn(T, H * xs).to(xdt)
          w = (torch.randn(H, N, K) / math.sqrt(K)).to(wdt)
          want = torch.einsum("thk,hnk->thn", x.double().view(T, H, xs)[..., :K], w.double())
          out = torch.full((T, H * os_), 9.0, dtype=odt, device=DEV)
          req = [0] * T
          req[T // 2] = -1
          ops.head_linear(x.to(DEV), xs, w.to(DEV), out, os_, ops.current_stream(), token_req=i32(req))
          got = out.double().cpu().view(T, H, os_)
          keep = [t for t in range(T) if t != T // 2]
          tol = 2e-5 * math.sqrt(K) if odt == torch.float32 else 3e-2
          assert float((got[keep][..., :N] - want[keep]).abs().max()) < tol, (wdt, xdt, odt)
          assert bool((got[..., N:] == 9.0).all()) and bool((got[T // 2] == 9.0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("D,n_mix", [(48, 5), (80, 1), (13, 3)])
def test_the_token_before_is_carried_from_step_to_step(act, D, n_mix):
    from mlx_lm_b200 import ops
    torch.manual_seed(D)
    T = 40
    x = torch.randn(2, T, D).to(act)
    mu = torch.rand(n_mix, D)
    x64 = x.double()
    before = torch.cat([torch.zeros(2, 1, D, dtype=torch.float64), x64[:, :-1]], dim=1)
    want = torch.stack([x64 + (before - x64) * mu[s].double() for s in range(n_mix)], dim=2)     # [2, T, n_mix, D]
    sec = (D + 7) // 8 * 8
    state = torch.full((3, D), 5.0, device=DEV)            # what an earlier request left in the slots
    slots = i32([2, 0])
    got = torch.zeros(2, T, n_mix, D, dtype=torch.float64)
    lo, cuts, i = 0, (1, 2, 1, 5, 3, 1, 17), 0
    while lo < T:
        n = min(cuts[i % len(cuts)], T - lo)
        xin = torch.cat([x[0, lo:lo + n], x[1, lo:lo + n]]).contiguous().to(DEV)
        out = torch.zeros(2 * n, n_mix * sec, dtype=act, device=DEV)
        ops.token_shift_mix(xin, mu.to(DEV), state, slots, i32(list(range(lo, lo + n)) * 2), i32([0] * n + [1] * n),
                            i32([0, n, 2 * n]), out, ops.current_stream())
        o = out.double().cpu().view(2, n, n_mix, sec)[..., :D]
        got[:, lo:lo + n] = o
        lo, i = lo + n, i + 1
    assert float((got - want).abs().max()) < (1e-6 if act == torch.float32 else 3e-2)
    assert float((state[2].double().cpu() - x64[0, -1]).abs().max()) == 0 and bool((state[1] == 5.0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,K", [(2, 32), (3, 48), (5, 16), (2, 128), (1, 7), (1, 200)])
def test_the_recurrence_with_a_data_dependent_decay(act, H, K):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * K)
    T, R = 50, 2
    sec = (H * K + 7) // 8 * 8
    rkv = torch.zeros(R, T, 3 * sec)
    rkv[..., :H * K], rkv[..., sec:sec + H * K], rkv[..., 2 * sec:2 * sec + H * K] = (torch.randn(3, R, T, H * K) * 0.5)
    rkv = rkv.to(act)
    d_raw = torch.randn(R, T, H * K) - 1.0
    u = torch.randn(H, K) * 0.5
    want = torch.zeros(R, T, H, K, dtype=torch.float64)
    S_end = torch.zeros(R, H, K, K, dtype=torch.float64)
    for r in range(R):
        rr, kk, vv = (rkv[r, :, i * sec:i * sec + H * K].double().view(T, H, K) for i in range(3))
        w = torch.exp(-torch.exp(d_raw[r].double())).view(T, H, K)
        for h in range(H):
            S = torch.zeros(K, K, dtype=torch.float64)
            for t in range(T):
                kv = torch.outer(kk[t, h], vv[t, h])
                want[r, t, h] = (S + u[h].double()[:, None] * kv).T @ rr[t, h]
                S = w[t, h][:, None] * S + kv
            S_end[r, h] = S
    state = torch.zeros(3, H, K, K, device=DEV)           # [slot, head, value column, key row]
    slots = i32([2, 0])
    got = torch.zeros(R, T, H * K, dtype=torch.float64)
    lo, cuts, i = 0, (1, 16, 2, 17, 1, 33), 0
    while lo < T:
        n = min(cuts[i % len(cuts)], T - lo)
        xin = torch.cat([rkv[0, lo:lo + n], rkv[1, lo:lo + n]]).contiguous().to(DEV)
        din = torch.cat([d_raw[0, lo:lo + n], d_raw[1, lo:lo + n]]).contiguous().to(DEV)
        o = torch.zeros(2 * n, H * K, device=DEV)
        ops.wkv_scan(xin, 0, sec, 2 * sec, din, u.to(DEV), state, slots, i32([0] * n + [1] * n), i32([0, n, 2 * n]), o, H,
                     ops.current_stream())
        got[0, lo:lo + n], got[1, lo:lo + n] = o[:n].double().cpu(), o[n:].double().cpu()
        lo, i = lo + n, i + 1
    scale = max(1.0, float(want.abs().max()))
    assert float((got.view(R, T, H, K) - want).abs().max()) < 1e-4 * scale
    for r, slot in ((0, 2), (1, 0)):
        assert float((state[slot].double().cpu().transpose(1, 2) - S_end[r]).abs().max()) < 1e-4 * max(1.0, float(S_end.abs().max()))
    assert float(state[1].abs().max()) == 0.0             # the slot nobody holds was not touched


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("F_", [64, 13])
def test_the_learned_activation(act, F_):
    from mlx_lm_b200 import ops
    torch.manual_seed(F_)
    x = (torch.randn(33, F_) * 3).to(act)
    numbers = torch.tensor([0.3, -0.7])
    want = plain.xielu(x.double(), numbers.double())
    xd = x.to(DEV)
    ops.xielu(xd, xd, numbers.to(DEV), ops.current_stream())
    err = (xd.double().cpu() - want).abs() / (1.0 + want.abs())
    assert float(err.max()) < (1e-6 if act == torch.float32 else 1e-2)


def test_tanh_in_a_product_s_epilogue():
    from mlx_lm_b200 import ops
    torch.manual_seed(0)
    for dtype, M in ((torch.float32, 9), (torch.bfloat16, 9), (torch.bfloat16, 200)):
        x, w = torch.randn(M, 64).to(dtype), (torch.randn(24, 64) / 8).to(dtype)
        out = torch.zeros(M, 24, dtype=dtype, device=DEV)
        from mlx_lm_b200.parts.linear import ACTIVATIONS
        if dtype == torch.float32:
            ops.linear_generic(x.to(DEV), w.to(DEV), None, out, ops.current_stream(), epilogue=ACTIVATIONS["tanh"])
        elif M <= ops.SMALL_M:
            ops.linear_few_rows(x.to(DEV), w.to(DEV), None, out, ops.current_stream(), epilogue=ACTIVATIONS["tanh"])
        else:
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            ops.linear_tensor_cores(x.to(DEV), w.to(DEV), None, out, status, ops.current_stream(), epilogue=ACTIVATIONS["tanh"])
        want = torch.tanh(x.double() @ w.double().T)
        assert float((out.double().cpu() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2)
