"""The kernels of the state-keeping layers and the norms of a float32 stream, each alone against the plain
functions of tests/plain_lelatar.py, with sequences cut into steps so that the state is carried."""
import pytest
import torch

import plain_lelatar as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
ACT = [torch.float32, torch.bfloat16]


def step_arrays(cuts_per_request, first_positions):
    """Device index arrays for one step: request r brings ``cuts_per_request[r]`` rows starting at its position."""
    token_req, positions, first_token = [], [], [0]
    for r, (n, p0) in enumerate(zip(cuts_per_request, first_positions)):
        token_req += [r] * n
        positions += list(range(p0, p0 + n))
        first_token.append(first_token[-1] + n)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    return i32(token_req), i32(positions), i32(first_token), i32(first_positions)


def run_in_steps(n_total, cuts, fn):
    """Call ``fn(lo, hi)`` over ``[0, n_total)`` cut as ``cuts`` (repeated)."""
    lo, i = 0, 0
    while lo < n_total:
        hi = min(n_total, lo + cuts[i % len(cuts)])
        fn(lo, hi)
        lo, i = hi, i + 1


@pytest.mark.parametrize("by_tap", [False, True])
@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("taps,C", [(4, 40), (2, 7), (3, 130), (4, 256)])
def test_short_convolution_carries_its_tail(act, taps, C, by_tap):
    from mlx_lm_b200 import ops
    torch.manual_seed(taps * C)
    T = 45
    x = torch.randn(2, T, C).to(act)
    w, b = torch.randn(C, taps) * 0.5, torch.randn(C) * 0.1
    want = torch.stack([plain.silu(plain.short_conv(x[r].double(), w.double(), b.double())) for r in range(2)])
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    state = torch.zeros(3, taps - 1, C, device=DEV)
    slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    got = torch.zeros(2, T, C, dtype=act, device=DEV)

    def step(lo, hi):
        n = hi - lo
        token_req, positions, first_token, first_pos = step_arrays([n, n], [lo, lo])
        xin = torch.cat([xd[0, lo:hi], xd[1, lo:hi]]).contiguous()
        out = torch.empty(2 * n, C, dtype=act, device=DEV)
        ops.conv_silu(xin, wd, bd, state, slots, positions, token_req, first_token, first_pos, out, ops.current_stream(),
                      weight_by_tap=wd.t().contiguous() if by_tap else None)
        got[0, lo:hi], got[1, lo:hi] = out[:n], out[n:]
    run_in_steps(T, (1, 2, 1, 5, 3, 1, 17), step)
    tol = 1e-5 if act == torch.float32 else 2e-2
    assert float((got.double().cpu() - want).abs().max()) < tol


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,G,N,V", [(4, 2, 24, 8), (2, 1, 16, 40), (6, 3, 70, 12), (1, 1, 3, 5)])
def test_state_space_scan(act, H, G, N, V):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * N + V)
    T = 50
    inner, GN = H * V, G * N
    xbc = (torch.randn(T, inner + 2 * GN) * 0.7).to(act)
    dt_raw = torch.randn(T, H).to(act)
    dt_bias, a_log, d_skip = torch.randn(H) * 0.5, torch.randn(H) * 0.5, torch.randn(H)
    # the plain recurrence
    x = xbc.double()[:, :inner].reshape(T, H, V)
    B = xbc.double()[:, inner:inner + GN].reshape(T, G, N)
    C = xbc.double()[:, inner + GN:].reshape(T, G, N)
    dt = plain.softplus(dt_raw.double() + dt_bias.double())
    a = torch.exp(-torch.exp(a_log.double()) * dt)
    grp = torch.arange(H) // (H // G)
    S = torch.zeros(H, N, V, dtype=torch.float64)
    want = torch.zeros(T, H, V, dtype=torch.float64)
    for t in range(T):
        S = a[t, :, None, None] * S + dt[t, :, None, None] * B[t, grp][:, :, None] * x[t, :, None, :]
        want[t] = torch.einsum("hnv,hn->hv", S, C[t, grp]) + d_skip.double()[:, None] * x[t]
    state = torch.zeros(2, H, V, N, device=DEV)          # the pool keeps a head's state column by column
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    got = torch.zeros(T, inner, device=DEV)
    xd, dd = xbc.to(DEV), dt_raw.to(DEV)

    def step(lo, hi):
        token_req, _, first_token, _ = step_arrays([hi - lo], [lo])
        y = torch.empty(hi - lo, inner, device=DEV)
        ops.mamba2_scan(xd[lo:hi], 0, inner, inner + GN, dd[lo:hi], dt_bias.to(DEV), a_log.to(DEV), d_skip.to(DEV), state,
                        slots, token_req, first_token, y, H, G, ops.current_stream())
        got[lo:hi] = y
    run_in_steps(T, (1, 16, 2, 17, 1, 33), step)
    assert float((got.double().cpu().reshape(T, H, V) - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))
    assert float((state[1].double().cpu().transpose(1, 2) - S).abs().max()) < 1e-4 * max(1.0, float(S.abs().max()))
    assert float(state[0].abs().max()) == 0.0          # the other slot was not touched


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,G,K,V", [(4, 2, 16, 24), (2, 2, 40, 8), (3, 1, 100, 20)])
def test_gated_delta_scan(act, H, G, K, V):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * K + V)
    T = 44
    qkv = torch.randn(T, 2 * G * K + H * V).to(act)
    b_raw, a_raw = torch.randn(T, H).to(act), torch.randn(T, H).to(act)
    dt_bias, a_log = torch.randn(H) * 0.5, torch.randn(H) * 0.5
    q = qkv.double()[:, :G * K].reshape(T, G, K)
    k = qkv.double()[:, G * K:2 * G * K].reshape(T, G, K)
    v = qkv.double()[:, 2 * G * K:].reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * K ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(b_raw.double())
    decay = torch.exp(-torch.exp(a_log.double()) * plain.softplus(a_raw.double() + dt_bias.double()))
    grp = torch.arange(H) // (H // G)
    S = torch.zeros(H, K, V, dtype=torch.float64)
    want = torch.zeros(T, H, V, dtype=torch.float64)
    for t in range(T):
        kt, qt = k[t, grp], q[t, grp]
        S = decay[t, :, None, None] * S
        u = beta[t, :, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        want[t] = torch.einsum("hkv,hk->hv", S, qt)
    state = torch.zeros(1, H, V, K, device=DEV)
    slots = torch.tensor([0], dtype=torch.int32, device=DEV)
    got = torch.zeros(T, H * V, device=DEV)
    qd, bd, ad = qkv.to(DEV), b_raw.to(DEV), a_raw.to(DEV)

    def step(lo, hi):
        token_req, _, first_token, _ = step_arrays([hi - lo], [lo])
        o = torch.empty(hi - lo, H * V, device=DEV)
        ops.gated_delta_scan(qd[lo:hi], 0, G * K, 2 * G * K, bd[lo:hi], ad[lo:hi], dt_bias.to(DEV), a_log.to(DEV), state,
                             slots, token_req, first_token, o, H, G, ops.current_stream())
        got[lo:hi] = o
    run_in_steps(T, (2, 1, 16, 1, 17), step)
    assert float((got.double().cpu().reshape(T, H, V) - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("act", ACT)
def test_rms_norms_and_the_stream_update(act):
    from mlx_lm_b200 import ops
    torch.manual_seed(0)
    R, D, eps = 9, 96, 1e-5
    x, g = torch.randn(R, D) * 3, torch.randn(R, D).to(act)
    s = ops.current_stream()
    tol = 1e-5 if act == torch.float32 else 1e-2     # of the largest value: bfloat16 rounds the result

    def close(a, b):
        return float((a - b).abs().max()) < tol * max(1.0, float(b.abs().max()))

    def run(**kw):
        out = torch.empty(R, D, dtype=act, device=DEV)
        w = kw.pop("weight")
        gate = kw.pop("gate", None)
        ops.rmsnorm(x.to(DEV), w.to(DEV), out, eps, s, gate=None if gate is None else gate.to(DEV), **kw)
        return out.double().cpu()

    w = torch.randn(D) * 0.1
    assert close(run(weight=w, offset=1.0), plain.norm_around_zero(x.double(), w.double(), eps))
    w4 = torch.randn(D)
    gated = x.double() * plain.silu(g.double())
    want = plain.unit_rms(gated.reshape(R, 4, D // 4), eps).reshape(R, D) * w4.double()
    assert close(run(weight=w4, groups=4, gate=g, gate_mode=ops.GATE_BEFORE), want)
    ws = torch.randn(D // 6)
    want = plain.unit_rms(x.double().reshape(R, 6, D // 6), eps) * ws.double()
    want = want.reshape(R, D) * plain.silu(g.double())
    assert close(run(weight=ws, groups=6, period=D // 6, gate=g, gate_mode=ops.GATE_AFTER), want)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, D, dtype=act, device=DEV)
    ops.rmsnorm(x.to(DEV), w.to(DEV), out, eps, s, offset=1.0, rows=rows)
    assert close(out.double().cpu(), plain.norm_around_zero(x.double()[[8, 0, 3]], w.double(), eps))
    # x += 0.5 * (norm(y1) w1 + norm(y2) w2), and a copy in the activation dtype
    y1, y2, w1, w2 = torch.randn(R, D), torch.randn(R, D) * 5, torch.randn(D), torch.randn(D)
    xd = x.to(DEV).clone()
    cast = torch.empty(R, D, dtype=act, device=DEV)
    ops.residual_update(xd, y1.to(DEV), s, w1=w1.to(DEV), y2=y2.to(DEV), w2=w2.to(DEV), scale=0.5, eps=eps, cast_out=cast)
    want = x.double() + 0.5 * (plain.norm_plain(y1.double(), w1.double(), eps) + plain.norm_plain(y2.double(), w2.double(), eps))
    assert float((xd.double().cpu() - want).abs().max()) < 1e-5
    assert close(cast.double().cpu(), want)


@pytest.mark.parametrize("M", [5, 37, 64, 100, 200])
def test_linear_kernels_add_a_float32_residual(M):
    """A float32 result takes a float32 residual (in place) in all three linear kernels."""
    from mlx_lm_b200 import ops
    torch.manual_seed(M)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    s = ops.current_stream()
    for N, K in ((72, 64), (16, 256), (200, 16)):
        x = torch.randn(M, K, device=DEV).bfloat16()
        w = (torch.randn(N, K, device=DEV) * K ** -0.5).bfloat16()
        res = torch.randn(M, N, device=DEV)
        want = res + x.float() @ w.float().T
        for kind in ("generic", "fast"):
            out = res.clone()
            if kind == "generic":
                ops.linear_generic(x, w, None, out, s, residual=out)
            elif M <= ops.SMALL_M:
                ops.linear_few_rows(x, w, None, out, s, residual=out)
            else:
                ops.linear_tensor_cores(x, w, None, out, status, s, residual=out)
            assert float((out - want).abs().max()) < 1e-3, (kind, M, N, K)
    assert int(status.item()) == 0
