"""CPU: the checker used for reduced-precision (TF32) training steps does what its contract says, on a stand-in
for the device: the same MLP step evaluated in float32 with operands rounded to 11 significant bits."""
import numpy as np


def _round_tf32(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x1000) & 0xFFFFE000          # round to nearest, ties away from zero, 10 explicit mantissa bits
    return u.astype(np.uint32).view(np.float32)


def _emulated_step(ws, bs, x, t):
    h, masks, hs = x, [], [x]
    for i, (w, b) in enumerate(zip(ws, bs)):
        z = _round_tf32(h) @ _round_tf32(w) + b
        if i + 1 < len(ws):
            masks.append(z > 0)
            z = np.maximum(z, 0)
        h = z.astype(np.float32)
        hs.append(h)
    g = (2.0 * (h - t) / h.size).astype(np.float32)
    gw, gb = [None] * len(ws), [None] * len(ws)
    for i in reversed(range(len(ws))):
        if i + 1 < len(ws):
            g = g * masks[i]
        gb[i] = g.sum(axis=0)
        gw[i] = _round_tf32(hs[i]).T @ _round_tf32(g)
        g = (_round_tf32(g) @ _round_tf32(ws[i]).T).astype(np.float32)
    return masks, gw, gb


def test_check_accepts_a_tf32_like_step_and_rejects_a_wrong_one(ora):
    rng = np.random.default_rng(0)
    dims, batch = [96, 160, 128, 24], 192
    ws = [rng.uniform(-np.sqrt(6 / dims[i]), np.sqrt(6 / dims[i]), (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.05).astype(np.float32) for i in range(3)]
    x, t = rng.standard_normal((batch, dims[0]), dtype=np.float32), rng.standard_normal((batch, dims[-1]), dtype=np.float32)
    masks, gw, gb = _emulated_step(ws, bs, x, t)
    chk = ora.reduced_precision_step_check(ws, bs, x, t, masks, gw, gb)
    assert chk["outside_mismatch"] == [0, 0]
    assert all(f <= 1e-3 * n for f, n in zip(chk["flips"], chk["elements"]))
    assert all(f <= b for f, b in zip(chk["flips"], chk["in_band"]))          # flips can only happen inside the band
    assert max(chk["rel_gw"]) <= 2e-3 and max(chk["rel_gb"]) <= 2e-3
    # with float64's own masks and gradients everything is exact
    exact = ora.mlp_step_f64(ws, bs, x, t)
    ok = ora.reduced_precision_step_check(ws, bs, x, t, [z > 0 for z in exact["z"][:2]], exact["gw"], exact["gb"])
    assert ok["flips"] == [0, 0] and max(ok["rel_gw"]) < 1e-12 and max(ok["rel_gb"]) < 1e-12
    # a gradient that is off by one percent, or a mask that is wrong away from zero, is caught
    bad = ora.reduced_precision_step_check(ws, bs, x, t, masks, [g * np.float32(1.01) for g in gw], gb)
    assert max(bad["rel_gw"]) > 2e-3
    wrong = [m.copy() for m in masks]
    far = np.argmax(np.abs(exact["z"][0]))
    wrong[0].reshape(-1)[far] ^= True
    assert ora.reduced_precision_step_check(ws, bs, x, t, wrong, gw, gb)["outside_mismatch"][0] == 1
