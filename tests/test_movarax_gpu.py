"""Movarax on the GPU against the plain implementation (tests/plain/movarax_plain.py): every mechanism alone, then
whole models through the engine: prompts, token-by-token decoding, unequal batches, slots used again, far keys and
page borders, captured graphs, and greedy generation through the library's entry point."""
import numpy as np
import pytest
import torch

import movarax_models as mm
from helpers import TraceRun, assert_logits
from plain import movarax_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(dtype).contiguous()


def host(t):
    return t.float().cpu().numpy()


def batch_of(sequences):
    """A filled StepBatch: sequences = [(slot, tokens or count, start)]."""
    from abacus_b200.engine.batch import Sequence, StepBatch
    sequences = [(slot, [0] * t if isinstance(t, int) else list(t), start) for slot, t, start in sequences]
    n = sum(len(t) for _, t, _ in sequences)
    b = StepBatch(n, len(sequences), 1, DEV)
    return b.fill([Sequence(slot, t, start, []) for slot, t, start in sequences], exact=True)


def latent_cache(row, rank, dtype, max_tokens=64 * 40):
    from abacus_b200.cache import CacheNeed, SequenceCache
    return SequenceCache([CacheNeed(n_kv_heads=1, head_dim=row, v_head_dim=rank, values_in_keys=True)], [None], max_tokens,
                         dtype, DEV)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,n,r,dims,R", [(2, 8, 8, 8, 16), (3, 10, 6, 4, 21), (1, 4, 16, 16, 24)])
def test_latent_prep_norms_rotates_and_writes_the_cache(dtype, H, n, r, dims, R):
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(H)
    row, eps, base = -(-(R + r) // 8) * 8, 1e-5, 300.0
    rnd = plain.bf16_round if dtype == "bfloat16" else (lambda a: a)
    cache = latent_cache(row, R, DT[dtype])
    slots = [cache.open_slot() for _ in range(3)]
    steps = [(slots[2], 70, 0), (slots[0], 3, 62)]            # one from its start over a page border, one further on
    for slot, count, start in steps:
        cache.reserve(slot, start + count)
    b = batch_of(steps)
    T = b.n_rows
    positions = np.concatenate([np.arange(start, start + count) for _, count, start in steps])
    down_at = -(-H * (n + r) // 8) * 8
    proj = np.zeros((T, down_at + R + r), dtype=np.float32)
    proj[:, :H * (n + r)] = rnd(rng.standard_normal((T, H * (n + r))))
    proj[:, down_at:] = rnd(rng.standard_normal((T, R + r)) * 3)
    w = (1.0 + rng.standard_normal(R) * 0.3).astype(np.float32)
    i = np.arange(dims // 2, dtype=np.float64)
    angle = np.arange(200, dtype=np.float64)[:, None] * np.power(base, -2.0 * i / dims)[None, :]
    cos, sin = dev(np.cos(angle)), dev(np.sin(angle))
    q_lat = torch.full((T, H * row), 7.0, dtype=DT[dtype], device=DEV)
    kv = cache.views[0].kv
    ops.latent_prep(dev(proj, DT[dtype]), down_at, H, n, r, R, dims, dev(w), eps, cos, sin, q_lat, row, R, False, kv, b)
    want_c = plain.norm(proj[:, down_at:down_at + R], w, eps)
    want_s = plain.rotate_pairs(proj[:, down_at + R:], positions, base, dims)
    q = proj[:, :H * (n + r)].reshape(T, H, n + r)
    want_q = plain.rotate_pairs(q[..., n:].transpose(1, 0, 2), positions, base, dims).transpose(1, 0, 2)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    table = kv.page_table.cpu().numpy()
    t = 0
    for slot, count, start in steps:
        for pos in range(start, start + count):
            got = host(kv.k[table[slot, pos // 64], 0, pos % 64])
            np.testing.assert_allclose(got[:R], want_c[t], **tol)
            np.testing.assert_allclose(got[R:R + r], want_s[t], **tol)
            assert not got[R + r:].any()
            t += 1
    got_q = host(q_lat).reshape(T, H, row)
    np.testing.assert_allclose(got_q[..., R:R + r], want_q, **tol)
    assert not got_q[..., R + r:].any() and (got_q[..., :R] == 7.0).all()   # the plain part is the product's to write
    # in full size: the whole head, plain part copied, into heads of n + r
    full = torch.zeros((T, H * (n + r) + 8), dtype=DT[dtype], device=DEV)
    ops.latent_prep(dev(proj, DT[dtype]), down_at, H, n, r, R, dims, None, eps, cos, sin, full, n + r, n, True, None, b)
    got = host(full)[:, :H * (n + r)].reshape(T, H, n + r)
    np.testing.assert_allclose(got[..., n:], want_q, **tol)
    np.testing.assert_array_equal(got[..., :n], q[..., :n])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,inner,outs", [(1, 3, 5, 7), (9, 2, 40, 16), (70, 4, 96, 33)])
def test_a_product_per_head(dtype, T, H, inner, outs):
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(T)
    rnd = plain.bf16_round if dtype == "bfloat16" else (lambda a: a)
    x_head, o_head = inner + 3, outs + 2
    x, w = rnd(rng.standard_normal((T, H * x_head + 1))), rnd(rng.standard_normal((H, outs, inner)))
    out = torch.full((T, H * o_head), 5.0, dtype=DT[dtype], device=DEV)
    ops.head_product(dev(x, DT[dtype]), x_head, dev(w, DT[dtype]), out, o_head, T)
    got = host(out).reshape(T, H, o_head)
    want = np.einsum("thi,hoi->tho", x[:, :H * x_head].reshape(T, H, x_head)[..., :inner], w)
    np.testing.assert_allclose(got[..., :outs], want, **(dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=1e-2, atol=3e-2)))
    assert (got[..., outs:] == 5.0).all()


def _latent_attention_want(q, rows, R, scale, sink):
    """q [T, H, row] at positions 0..T-1 over cache rows [T, row] whose first R elements are the values."""
    out = np.zeros((q.shape[0], q.shape[1], R))
    for a in range(q.shape[1]):
        out[:, a] = plain.softmax_with_sink((q[:, a].astype(np.float64) @ rows.T.astype(np.float64)) * scale, sink[a]) @ rows[:, :R]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,row,R", [(2, 24, 16), (5, 112, 96), (20, 40, 33), (16, 64, 48), (32, 96, 80), (3, 168, 160), (8, 256, 192)])
def test_attention_over_latent_rows_finds_one_loud_key_wherever_it_is(dtype, H, row, R):
    """A query that matches one key far more than the others: far back, at the sequence's start, on both sides of page
    borders, the token itself; the prompt in one step, and a token alone against a cache in a slot that was used before."""
    from abacus_b200.kernels import ops
    from abacus_b200.parts import Workspace
    rng = np.random.default_rng(row)
    rnd = plain.bf16_round if dtype == "bfloat16" else (lambda a: a)
    T, scale = 200, 0.5
    cache = latent_cache(row, R, DT[dtype])
    first = cache.open_slot()
    cache.reserve(first, 64 * 5)
    kv = cache.views[0].kv
    kv.k.fill_(9.0)                      # whatever the slot's last user left
    cache.close_slot(first)
    other, slot = cache.open_slot(), cache.open_slot()
    cache.reserve(other, 30), cache.reserve(slot, T)
    rows = rnd(rng.standard_normal((T, row)) * 0.3).astype(np.float32)
    sink = rng.standard_normal(H).astype(np.float32)
    table = kv.page_table.cpu().numpy()
    for pos in range(T):
        kv.k[table[slot, pos // 64], 0, pos % 64] = dev(rows[pos], DT[dtype])
    ws = Workspace(torch.device(DEV, torch.cuda.current_device()))
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
    for loud in (0, 1, 63, 64, 65, 127, 128, 198, 199):
        q = rnd(rng.standard_normal((T, H, row)) * 0.3).astype(np.float32)
        q[-1] += rnd(rows[loud] * 40.0 / (rows[loud] ** 2).sum())[None, :]       # the last token looks for `loud`
        want = _latent_attention_want(q, rows, R, scale, sink)
        p = plain.softmax_with_sink((q[:, 0].astype(np.float64) @ rows.T.astype(np.float64)) * scale, sink[0])
        assert p[-1, loud] > 0.9
        # the whole prompt as one step (the general kernel), then the last token alone (split along the keys)
        out = torch.empty((T, H * R), dtype=DT[dtype], device=DEV)
        ops.attention_values_in_keys(dev(q.reshape(T, -1), DT[dtype]), out, H, row, R, scale, batch_of([(slot, T, 0)]), kv, dev(sink), ws)
        np.testing.assert_allclose(host(out).reshape(T, H, R), want, **tol)
        one = torch.empty((2, H * R), dtype=DT[dtype], device=DEV)
        b = batch_of([(other, 1, 29), (slot, 1, T - 1)])
        ops.attention_values_in_keys(dev(np.stack([q[29], q[-1]]).reshape(2, -1), DT[dtype]), one, H, row, R, scale, b, kv, dev(sink), ws)
        np.testing.assert_allclose(host(one)[1].reshape(H, R), want[-1], **tol)


@pytest.mark.parametrize("form", ["token by token", "chunks"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,n,V", [(2, 5, 3), (3, 16, 8), (1, 40, 24), (2, 128, 70), (1, 200, 133)])
def test_the_recurrence_whole_in_portions_token_by_token_and_in_an_unequal_batch(dtype, H, n, V, form):
    """Both kernels: the recurrence as it stands (decode steps) and in chunks of 64 tokens (steps that bring prompts)."""
    from abacus_b200.cache import CacheNeed, SequenceCache
    from abacus_b200.kernels import ops
    from abacus_b200.parts import Workspace
    ws = Workspace(torch.device(DEV, torch.cuda.current_device()))
    rng = np.random.default_rng(n)
    rnd = plain.bf16_round if dtype == "bfloat16" else (lambda a: a)
    decay = [0.995, 0.6, 1.0][:H]
    cache = SequenceCache([CacheNeed(states=(("decay_state", (H, n, V), "float32"),))], [None], 64, DT[dtype], DEV, max_slots=6)
    state = cache.views[0].states["decay_state"]
    lens = [150, 1, 70]
    at_k, at_v = H * n + 3, 2 * H * n + 8
    width = at_v + H * V + 1
    seqs = [rnd(rng.standard_normal((t, width)) * 1.5).astype(np.float32) for t in lens]

    def want_of(x):
        q = plain.silu(x[:, :H * n]).reshape(-1, H, n)
        k, v = plain.silu(x[:, at_k:at_k + H * n]).reshape(-1, H, n), plain.silu(x[:, at_v:at_v + H * V]).reshape(-1, H, V)
        return np.stack([plain.decay_recurrence(q[:, a].astype(np.float64), k[:, a].astype(np.float64), v[:, a].astype(np.float64),
                                                decay[a]) for a in range(H)], axis=1).reshape(-1, H * V)
    want = [want_of(x) for x in seqs]
    tol = dict(rtol=3e-5, atol=3e-5 * max(1.0, float(np.abs(np.concatenate(want)).max())))

    def run(steps):
        """steps: [[(sequence, first row, end row)]]; slots are opened as sequences appear. Returns the outputs by sequence."""
        slots, got = {}, {i: [] for i in range(len(seqs))}
        for step in steps:
            for i, a, z in step:
                if i not in slots:
                    slots[i] = cache.open_slot()
            b = batch_of([(slots[i], z - a, a) for i, a, z in step])
            x = np.concatenate([seqs[i][a:z] for i, a, z in step])
            out = torch.empty((len(x), H * V), dtype=torch.float32, device=DEV)
            if form == "chunks":
                ops.lightning_chunks(dev(x, DT[dtype]), 0, at_k, at_v, H, n, V, dev(np.array(decay)), state, out, b, ws)
            else:
                ops.lightning_scan(dev(x, DT[dtype]), 0, at_k, at_v, H, n, V, dev(np.array(decay)), state, out, b)
            row = 0
            for i, a, z in step:
                got[i].append(host(out[row:row + z - a]))
                row += z - a
        for slot in slots.values():
            cache.close_slot(slot)
        return [np.concatenate(got[i]) for i in range(len(seqs))]
    state.fill_(3.0)   # a slot's state is zeroed when the slot is handed out, whatever its last user left
    for what, steps in (("each whole, one batch", [[(0, 0, 150), (1, 0, 1), (2, 0, 70)]]),
                        ("portions down to two tokens", [[(0, 0, 67), (2, 0, 2)], [(0, 67, 131), (1, 0, 1), (2, 2, 70)], [(0, 131, 133)], [(0, 133, 150)]]),
                        ("token by token", [[(0, t, t + 1)] + ([(2, t, t + 1)] if t < 70 else []) + ([(1, 0, 1)] if t == 4 else []) for t in range(150)])):
        for i, (g, w) in enumerate(zip(run(steps), want)):
            np.testing.assert_allclose(g, w, err_msg=f"{what}, sequence {i}", **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_gated_norm_over_a_whole_row(dtype):
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(0)
    T, width, eps = 5, 173, 1e-5
    rnd = plain.bf16_round if dtype == "bfloat16" else (lambda a: a)
    o, w = rng.standard_normal((T, width)).astype(np.float32) * 4, (1 + rng.standard_normal(width) * 0.2).astype(np.float32)
    gate = rnd(rng.standard_normal((T, width + 4))).astype(np.float32)
    out = torch.empty((T, width), dtype=DT[dtype], device=DEV)
    ops.gated_row_norm(dev(o), dev(gate, DT[dtype])[:, 2:], dev(w), out, eps, batch_of([(0, 4, 0), (1, 1, 9)]))
    want = plain.norm(o, w, eps) * plain.sigmoid(gate[:, 2:2 + width])
    np.testing.assert_allclose(host(out), want, **(dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,d,ff", [(5, 2, 64, 24), (1, 1, 32, 8), (3, 3, 48, 16), (64, 6, 40, 9)])
def test_the_router_and_the_products_by_expert(dtype, E, top, d, ff):
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(E)
    rnd = plain.bf16_round if dtype == "bfloat16" else (lambda a: a)
    T = 37
    h = rnd(rng.standard_normal((T, d))).astype(np.float32)
    p = {"router": (rng.standard_normal((E, d)) * 0.5).astype(np.float32)}
    p["router"][E // 2] = p["router"][0]                         # a tie: the lower index wins
    for e in range(E):
        p[f"e{e}.up"], p[f"e{e}.down"] = rnd(rng.standard_normal((ff, d)) * 0.3), rnd(rng.standard_normal((d, ff)) * 0.3)
    b = batch_of([(0, 30, 0), (1, 7, 5)])
    expert = torch.empty(T * top, dtype=torch.int32, device=DEV)
    weight = torch.empty(T * top, dtype=torch.float32, device=DEV)
    x = dev(h, DT[dtype])
    ops.moe_route(x, dev(p["router"]), top, b, expert, weight)
    chosen, scores = plain.route(h, p["router"], top)
    np.testing.assert_array_equal(expert.cpu().numpy().reshape(T, top), chosen)
    np.testing.assert_allclose(weight.cpu().numpy().reshape(T, top), scores, rtol=1e-5, atol=1e-6)
    up = dev(np.stack([p[f"e{e}.up"] for e in range(E)]), DT[dtype])
    down = dev(np.stack([p[f"e{e}.down"] for e in range(E)]), DT[dtype])
    act = torch.empty((T * top, ff), dtype=DT[dtype], device=DEV)
    ops.routed_product(x, top, up, expert, weight, act, T * top, activation=ops.RELU_SQUARED)
    pair_out = torch.empty((T * top, d), dtype=torch.float32, device=DEV)
    ops.routed_product(act, 1, down, expert, None, pair_out, T * top)
    out = dev(np.ones((T, d)))
    ops.moe_combine(pair_out, out, T, top, add=True)
    want = 1.0 + plain.routed_feed_forward(h, p, {"router": {"experts": E, "top": top}}, None if dtype == "float32" else plain.bf16_round)
    np.testing.assert_allclose(host(out), want, **(dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)))
    ops.moe_combine(pair_out, out, T, top, add=False)
    np.testing.assert_allclose(host(out), want - 1.0, **(dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)))
    if ops.grouped_takes(x, up, down):
        # the same over rows sorted by expert, on the tensor cores: an expert's run of rows padded to whole tiles
        tiles = ops.grouped_tiles(T * top, E)
        scratch = torch.empty(2 * E + T * top, dtype=torch.int32, device=DEV)
        place, tile_expert = torch.empty(T * top, dtype=torch.int32, device=DEV), torch.empty(tiles, dtype=torch.int32, device=DEV)
        rows = torch.full((tiles * 128, d), float("nan"), dtype=DT[dtype], device=DEV)   # (padding rows hold anything)
        ops.moe_sort(x, top, expert, weight, T * top, E, scratch, place, tile_expert, rows)
        places = place.cpu().numpy()
        assert len(set(places.tolist())) == T * top and (tile_expert.cpu().numpy()[places // 128] == chosen.reshape(-1)).all()
        act2 = torch.empty((tiles * 128, ff), dtype=DT[dtype], device=DEV)
        ops.gemm_grouped(rows, up, act2, tile_expert, activation=ops.RELU_SQUARED)
        sorted_out = torch.empty((tiles * 128, d), dtype=torch.float32, device=DEV)
        ops.gemm_grouped(act2, down, sorted_out, tile_expert)
        out2 = dev(np.ones((T, d)))
        ops.moe_unsort(sorted_out, place, out2, T, top, add=True)
        np.testing.assert_allclose(host(out2), want, rtol=2e-2, atol=2e-2)
        ops.moe_unsort(sorted_out, place, out2, T, top, add=False)
        np.testing.assert_allclose(host(out2), want - 1.0, rtol=2e-2, atol=2e-2)
        assert not ops.kernel_status(x.device).any()
    sq = dev(h, DT[dtype])
    ops.relu_squared(sq, T)
    np.testing.assert_allclose(host(sq), rnd(plain.relu_squared(h)), rtol=1e-6, atol=1e-6)


# ------------------------------------------------------------------ whole models through the engine
def _engine(tmp_path, name, dtype, **kw):
    from abacus_b200.engine import Engine, load_model
    folder, raw, tensors = mm.write_folder(tmp_path, name)
    model = load_model(folder, dtype)
    return Engine(model, **{"max_tokens": 64 * 24, **kw}), raw, tensors, folder


def _full_size(raw, dtype):
    """Per latent layer: whether a bfloat16 prompt from its first token makes keys and values in full size (sizes the
    prompt kernel for ordinary heads takes); all other rows go over the cache's latent rows."""
    out = {}
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            head = m["dim"] + m["rot_dim"]
            out[i] = (dtype == "bfloat16" and head % 8 == 0 and head <= 256 and m["vdim"] % 8 == 0 and 8 <= m["vdim"] <= 128
                      and m["kv_rank"] % 8 == 0)
    return out


def _oracle(raw, tensors, tokens, dtype, prompt=None):
    """(plain logits in the engine's manner, the noise to allow for). prompt: how many tokens came as one step from
    the sequence's start (default all); the rest came one by one."""
    prompt = len(tokens) if prompt is None else prompt
    rows = {i: np.array([not (full and t < prompt) for t in range(len(tokens))]) for i, full in _full_size(raw, dtype).items()}
    if dtype == "float32":
        want = plain.forward(raw, tensors, tokens)
        return want, float(np.abs(want - plain.forward(raw, tensors, tokens, real=np.float64)).max())
    want = plain.forward(raw, tensors, tokens, rnd=plain.bf16_round, latent_rows=rows)
    return want, float(np.abs(want - plain.forward(raw, tensors, tokens)).max())


@pytest.mark.parametrize("name,dtype", [("U", "float32"), ("V", "float32"), ("W", "float32"),
                                        ("U", "bfloat16"), ("V", "bfloat16"), ("W", "bfloat16")])
def test_prompts_decoding_batches_and_used_slots_against_the_plain_model(tmp_path, name, dtype):
    engine, raw, tensors, _ = _engine(tmp_path, name, dtype)
    rng = np.random.default_rng(7)
    vocab = raw["vocab"]
    lens = [150, 1, 37, 80]
    seqs = [[int(t) for t in rng.integers(0, vocab, n)] for n in lens]
    # each alone, whole, all logits wanted; the slot is given back and used again by the next
    for s in seqs:
        want, noise = _oracle(raw, tensors, s, dtype)
        slot = engine.open()
        got = engine.step([(slot, s, list(range(len(s))))]).cpu().numpy()
        engine.close(slot)
        assert_logits(got, want, dtype, f"{name} whole, {len(s)} tokens", noise)
    # together in one batch of unequal prompts, cut before their ends, then decoded together; early enders leave
    cut = [100, 1, 20, 64]
    oracle = [_oracle(raw, tensors, s, dtype, prompt=c) for s, c in zip(seqs, cut)]
    slots = [engine.open() for _ in seqs]
    got = engine.step([(slot, s[:c], [c - 1]) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    for i, (want, noise) in enumerate(oracle):
        assert_logits(got[i:i + 1], want[cut[i] - 1:cut[i]], dtype, f"{name} batch prompt {i}", noise)
    step = 0
    while True:
        live = [i for i in range(len(seqs)) if cut[i] + step < len(seqs[i])]
        for i in range(len(seqs)):
            if cut[i] + step == len(seqs[i]) and slots[i] is not None:
                engine.close(slots[i])
                slots[i] = None
        if not live:
            break
        got = engine.step([(slots[i], [seqs[i][cut[i] + step]], [0]) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            assert_logits(got[j:j + 1], oracle[i][0][cut[i] + step:cut[i] + step + 1], dtype,
                          f"{name} batch decode, request {i}, position {cut[i] + step}", oracle[i][1])
        step += 1
    engine.check_status()


@pytest.mark.parametrize("name", ["U", "V"])
def test_portions_of_a_prompt_give_the_whole_prompts_logits(tmp_path, name):
    """A prompt cut into steps of several sizes, down to two tokens, beside another sequence that decodes."""
    engine, raw, tensors, _ = _engine(tmp_path, name, "float32")
    rng = np.random.default_rng(5)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 140)]
    want, noise = _oracle(raw, tensors, tokens, "float32")
    slot = engine.open()
    got, at = [], 0
    for size in (60, 2, 7, 1, 64, 6):
        got.append(engine.step([(slot, tokens[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    engine.close(slot)
    assert at == len(tokens)
    assert_logits(np.concatenate(got), want, "float32", f"{name} in portions", noise)


@pytest.mark.parametrize("name", ["U", "W"])
def test_token_by_token_from_the_first_token_and_long_decoding(tmp_path, name):
    """No prompt at all: every token a step of its own, over three pages."""
    engine, raw, tensors, _ = _engine(tmp_path, name, "float32")
    rng = np.random.default_rng(3)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 200)]
    want, noise = _oracle(raw, tensors, tokens, "float32")
    slot = engine.open()
    got = np.concatenate([engine.step([(slot, [t], [0])]).cpu().numpy() for t in tokens])
    engine.close(slot)
    assert_logits(got, want, "float32", f"{name} token by token", noise)


def test_a_far_token_decides_the_answer_through_both_mixers(tmp_path):
    """The same long prompts but for one early token: the last position's logits must follow the plain model's, which
    move (the latent cache reaches back over pages; a head with decay 0.99 and one with 0.97 still carry the token)."""
    engine, raw, tensors, _ = _engine(tmp_path, "U", "float32")
    rng = np.random.default_rng(9)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 190)]
    other = list(tokens)
    other[3] = (tokens[3] + 1) % raw["vocab"]
    wants = [plain.forward(raw, tensors, t)[-1] for t in (tokens, other)]
    assert np.abs(wants[0] - wants[1]).max() > 1e-3
    for t, want in zip((tokens, other), wants):
        slot = engine.open()
        engine.step([(slot, t[:130], [])])
        for tok in t[130:-1]:
            engine.step([(slot, [tok], [])])
        got = engine.step([(slot, t[-1:], [0])]).cpu().numpy()[0]
        engine.close(slot)
        assert np.abs(got - want).max() < 0.05 * np.abs(wants[0] - wants[1]).max() + 2e-4


def test_graphs_and_plain_launches_give_the_same_bits_and_states_survive_a_capture(tmp_path):
    from abacus_b200.engine import Engine
    engine, raw, tensors, _ = _engine(tmp_path, "U", "float32")
    eager = Engine(engine.model, max_tokens=64 * 24, use_graphs=False)
    rng = np.random.default_rng(11)
    seqs = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (30, 9)]
    outs = []
    for e in (engine, eager):
        slots = [e.open() for _ in seqs]
        got = [e.step([(slot, s[:5], [4]) for slot, s in zip(slots, seqs)]).cpu().numpy()]
        for i in range(5, 9):
            got.append(e.step([(slot, [s[i]], [0]) for slot, s in zip(slots, seqs)]).cpu().numpy())
        for i in range(9, 30):  # the second has ended: another graph (one row) is captured in mid-sequence
            got.append(e.step([(slots[0], [seqs[0][i]], [0])]).cpu().numpy())
        for slot in slots:
            e.close(slot)
        outs.append(np.concatenate(got))
    assert engine.graphs is not None and engine.graphs.graphs, "the engine did not replay captured graphs"
    np.testing.assert_array_equal(outs[0], outs[1])


def test_greedy_generation_through_the_entry_point(tmp_path):
    from abacus_b200 import LM
    folder, raw, tensors = mm.write_folder(tmp_path, "U")
    lm = LM(folder, dtype="float32", max_tokens=64 * 16)
    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (12, 3, 30)]
    outs = lm.generate(prompts, max_new_tokens=20, temperature=0.0, stop_tokens=[])
    for p, out in zip(prompts, outs):
        assert len(out) == 20
        logits = plain.forward(raw, tensors, p + out)
        for i, t in enumerate(out):  # each token is the plain model's choice, or within rounding of it
            row = logits[len(p) + i - 1]
            assert row[t] >= row.max() - 1e-3, f"token {i}: the engine chose {t}, the plain model {int(row.argmax())}"
    again = lm.generate(prompts[::-1], max_new_tokens=20, temperature=0.0, stop_tokens=[], batch_size=2)
    assert again == outs[::-1]


def test_trace_replay_of_a_model_folder(tmp_path):
    folder, raw, tensors = mm.write_folder(tmp_path, "V")
    rng = np.random.default_rng(4)
    a, b = ([int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (70, 9))
    run = TraceRun(folder, "float32", tmp_path / "out", 64 * 8)
    got = run.step([("a", a[:66], [0, 65]), ("b", b[:8], [7])]).reshape(3, -1)
    more = [run.step([("a", [a[66 + i]], [0])] + ([("b", [b[8]], [0])] if i == 0 else []), end=["b"] if i == 0 else []) for i in range(4)]
    run.step([], end=["a"])
    run.close()
    wa, wb = plain.forward(raw, tensors, a), plain.forward(raw, tensors, b)
    noise = float(np.abs(wa - plain.forward(raw, tensors, a, real=np.float64)).max())
    assert_logits(got, np.stack([wa[0], wa[65], wb[7]]), "float32", "replayed prompt", noise)
    assert_logits(more[0].reshape(2, -1), np.stack([wa[66], wb[8]]), "float32", "replayed decode", noise)
    assert_logits(np.stack([m.reshape(-1, raw["vocab"])[0] for m in more[1:]]), wa[67:70], "float32", "replayed decode", noise)
