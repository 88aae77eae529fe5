"""Temetar on the GPU against the plain implementation (tests/plain/temetar_plain.py): every mechanism alone, then
whole models through the engine: prompts, token-by-token decoding, unequal batches, slots used again, windows and
page borders, captured graphs, and greedy generation through the library's entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import temetar_models as tm
from helpers import ROOT, TRACE_RUN, TraceRun, assert_logits
from plain import temetar_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(dtype).contiguous()


def batch_of(sequences, plans=()):
    """A filled StepBatch: sequences = [(slot, tokens, start)]."""
    from abacus_b200.engine.batch import Sequence, StepBatch
    n = sum(len(t) for _, t, _ in sequences)
    b = StepBatch(n, len(sequences), 1, DEV, plans=plans)
    return b.fill([Sequence(slot, list(t), start, []) for slot, t, start in sequences], exact=True)


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("s,d", [(1, 40), (3, 64), (8, 300)])
def test_streams_step_writes_reads_and_norms(s, d):
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(s)
    T, m, eps = 7, 0.7, 1e-5
    X = rng.standard_normal((s, T, d)).astype(np.float32)
    y = rng.standard_normal((T, d)).astype(np.float32)
    M, c, a = (rng.standard_normal((s, s)).astype(np.float32), rng.standard_normal(s).astype(np.float32),
               rng.standard_normal(s).astype(np.float32))
    w = (rng.standard_normal(d) * 0.1).astype(np.float32)
    X2 = plain.streams_write(X, y, M, c, np.float32(m))
    want = plain.norm_one_plus(plain.streams_read(X2, a), w, eps)
    x = dev(X.transpose(1, 0, 2))
    out = torch.empty((T, d), dtype=torch.float32, device=DEV)
    ops.streams_step(x, dev(y), (dev(M), dev(c)), m, dev(a), dev(1 + w), eps, out)
    np.testing.assert_allclose(x.cpu().numpy().transpose(1, 0, 2), X2, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=5e-5, atol=5e-5)
    # nothing pending: the streams stay, the read is of the old ones; no norm: the read itself
    x = dev(X.transpose(1, 0, 2))
    ops.streams_step(x, None, None, 0.0, dev(a), None, 0.0, out)
    np.testing.assert_array_equal(x.cpu().numpy().transpose(1, 0, 2), X)
    np.testing.assert_allclose(out.cpu().numpy(), plain.streams_read(X, a), rtol=2e-5, atol=2e-5)
    # chosen rows: the sum of the new streams, normed, and the streams are left alone
    rows = torch.tensor([5, 0, 2], dtype=torch.int32, device=DEV)
    picked = torch.empty((3, d), dtype=torch.float32, device=DEV)
    ops.streams_step(x, dev(y), (dev(M), dev(c)), m, dev(np.ones(s)), dev(1 + w), eps, picked, rows=rows)
    np.testing.assert_array_equal(x.cpu().numpy().transpose(1, 0, 2), X)
    np.testing.assert_allclose(picked.cpu().numpy(), plain.norm_one_plus(X2.sum(0), w, eps)[[5, 0, 2]], rtol=5e-5, atol=5e-5)


def test_embedding_with_the_pair_table_remembers_the_last_token_of_a_step():
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(0)
    vocab, d, buckets, s = 50, 24, 11, 2
    table, pairs = rng.standard_normal((vocab, d)).astype(np.float32), rng.standard_normal((buckets + 1, d)).astype(np.float32)
    hashing = {"buckets": buckets, "mul_prev": 5, "mul_cur": 9}
    seqs = {3: [int(t) for t in rng.integers(0, vocab, 9)], 0: [int(t) for t in rng.integers(0, vocab, 4)]}
    want = {slot: plain.embedding(t, table, 1.5, pairs, hashing) for slot, t in seqs.items()}
    remembered = torch.full((4,), 49, dtype=torch.int32, device=DEV)  # stale tokens of the slots' last users
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = {slot: [] for slot in seqs}
    # slot 3: 5 tokens, then 1, then 3; slot 0: 1 token (a first token alone), then 3
    for step in ([(3, 0, 5), (0, 0, 1)], [(3, 5, 6), (0, 1, 4)], [(3, 6, 9)]):
        b = batch_of([(slot, seqs[slot][a:z], a) for slot, a, z in step])
        x = torch.empty((b.n_rows, s, d), dtype=torch.float32, device=DEV)
        ops.embed_pairs(b, dev(table), dev(pairs), remembered, x, 1.5, buckets, 5, 9, status)
        ops.remember_tokens(b, remembered)
        at = 0
        for slot, a, z in step:
            got[slot].append(x[at:at + z - a].cpu().numpy())
            at += z - a
    for slot in seqs:
        g = np.concatenate(got[slot])
        np.testing.assert_allclose(g[:, 0], want[slot], rtol=1e-6, atol=1e-6)
        np.testing.assert_array_equal(g[:, 0], g[:, 1])  # every stream starts as the same copy
    assert status.tolist() == [0, 0, 0, 0] and remembered.tolist()[3] == seqs[3][-1] and remembered.tolist()[0] == seqs[0][-1]


@pytest.mark.parametrize("taps,C", [(1, 37), (2, 37), (4, 37), (3, 40), (8, 48)])
def test_short_convolution_in_portions_of_every_size(taps, C):
    """37 channels go one to a thread, 40 and 48 several to a thread as one vector."""
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(taps)
    ld, T = 48, 23
    x = rng.standard_normal((T, ld)).astype(np.float32)
    w = rng.standard_normal((C, taps)).astype(np.float32)
    want = plain.silu(plain.short_convolution(x[:, :C], w))
    tail = torch.randn((3, max(taps - 1, 0), C), device=DEV)  # what the slot's last user left
    tail[2].zero_()  # a slot is zeroed when it is handed out
    got, at = [], 0
    for n in (5, 2, 1, 1, 3, 2, 9):  # portions down to one token, shorter than the taps and longer
        b = batch_of([(2, [0] * n, at)])
        out = torch.empty((n, C), dtype=torch.float32, device=DEV)
        xin = dev(x[at:at + n])
        ops.short_conv(xin, C, dev(w), tail, out, b, update_tail=n == 1)  # one token: the kernel moves the tail itself
        if n > 1:
            ops.short_conv_tail(xin, C, taps, tail, b)
        got.append(out.cpu().numpy())
        at += n
    np.testing.assert_allclose(np.concatenate(got), want, rtol=2e-5, atol=2e-5)


def _delta_inputs(rng, T, H, G, K, V):
    qkv = rng.standard_normal((T, 2 * G * K + H * V)).astype(np.float32)
    decay_in = rng.standard_normal((T, H * K)).astype(np.float32)
    beta_in = rng.standard_normal((T, H + 3)).astype(np.float32)
    a_log, bias = (rng.standard_normal(H) * 0.5 - 1).astype(np.float32), (rng.standard_normal(H * K) * 0.5).astype(np.float32)
    return qkv, decay_in, beta_in, a_log, bias


def _delta_plain(qkv, decay_in, beta_in, a_log, bias, H, G, K, V, real=np.float32):
    T = qkv.shape[0]
    qkv, decay_in, beta_in, a_log, bias = (t.astype(real) for t in (qkv, decay_in, beta_in, a_log, bias))
    q = plain.unit_vectors(qkv[:, :G * K].reshape(T, G, K)) * real(K) ** real(-0.5)
    k = plain.unit_vectors(qkv[:, G * K:2 * G * K].reshape(T, G, K))
    q, k = np.repeat(q, H // G, axis=1), np.repeat(k, H // G, axis=1)
    g = np.exp(-np.exp(a_log)[None, :, None] * plain.softplus(decay_in + bias).reshape(T, H, K))
    return plain.delta_recurrence(q, k, qkv[:, 2 * G * K:].reshape(T, H, V), g, plain.sigmoid(beta_in[:, :H])).reshape(T, H * V)


@pytest.mark.parametrize("H,G,K,V", [(2, 2, 32, 48), (4, 2, 16, 8), (3, 1, 40, 20), (2, 1, 72, 40), (1, 1, 256, 130), (2, 2, 5, 3)])
def test_delta_rule_whole_in_portions_and_token_by_token(H, G, K, V):
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(K)
    T = 45
    ins = _delta_inputs(rng, T, H, G, K, V)
    want = _delta_plain(*ins, H, G, K, V)
    noise = np.abs(want - _delta_plain(*ins, H, G, K, V, real=np.float64)).max()
    qkv, decay_in, beta_in, a_log, bias = ins
    from abacus_b200.parts import Workspace
    ws = Workspace(torch.device(DEV, torch.cuda.current_device()))
    for cuts in ([T], [17, 2, 1, 25], [1] * T):
        state = torch.randn((3, H, V, K), device=DEV)
        state[1].zero_()
        got, at = [], 0
        for n in cuts:
            b = batch_of([(1, [0] * n, at)])
            out = torch.empty((n, H * V), dtype=torch.float32, device=DEV)
            ops.delta_scan(dev(qkv[at:at + n]), dev(decay_in[at:at + n]), dev(beta_in[at:at + n])[:, :H + 3], dev(a_log),
                           dev(bias), state, out, b, H, G, K, V, ws)
            got.append(out.cpu().numpy())
            at += n
        np.testing.assert_allclose(np.concatenate(got), want, rtol=1e-4, atol=2e-5 + 4 * noise, err_msg=str(cuts[:4]))


def test_delta_rule_in_an_unequal_batch_and_in_bfloat16_inputs():
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(5)
    H, G, K, V = 4, 2, 48, 24
    lens, slots = [33, 1, 18], [2, 0, 5]
    ins = [_delta_inputs(rng, n, H, G, K, V) for n in lens]
    ins = [(plain.bf16_round(a), b, plain.bf16_round(c), d, e) for a, b, c, d, e in ins]
    want = [_delta_plain(*i, H, G, K, V) for i in ins]
    a_log, bias = ins[0][3], ins[0][4]
    want = [_delta_plain(i[0], i[1], i[2], a_log, bias, H, G, K, V) for i in ins]
    state = torch.zeros((6, H, V, K), device=DEV)
    b = batch_of([(slot, [0] * n, 0) for slot, n in zip(slots, lens)])
    cat = lambda j: np.concatenate([i[j] for i in ins])
    out = torch.empty((sum(lens), H * V), dtype=torch.float32, device=DEV)
    from abacus_b200.parts import Workspace
    ops.delta_scan(dev(cat(0), torch.bfloat16), dev(cat(1)), dev(cat(2), torch.bfloat16), dev(a_log), dev(bias), state, out,
                   b, H, G, K, V, Workspace(torch.device(DEV, torch.cuda.current_device())))
    np.testing.assert_allclose(out.cpu().numpy(), np.concatenate(want), rtol=1e-4, atol=5e-5)
    assert float(state[1].abs().max()) == 0.0 and float(state[2].abs().max()) > 0.0  # only the step's slots are touched


def test_gated_head_norm():
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(1)
    T, H, V, eps = 9, 3, 20, 1e-5
    o, gate = rng.standard_normal((T, H * V)).astype(np.float32), rng.standard_normal((T, H * V)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(V)).astype(np.float32)
    want = (plain.norm_plain(o.reshape(T, H, V), w, eps) * plain.sigmoid(gate.reshape(T, H, V))).reshape(T, H * V)
    out = torch.empty((T, H * V), dtype=torch.float32, device=DEV)
    ops.gated_head_norm(dev(o), dev(gate), dev(w), out, T, H, V, eps)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-5, atol=2e-5)


def _attention_case(T, H, G, D, V, window, keep, scale, loud=None, seed=0):
    """q, k, v of one sequence and the plain result. loud = (query position, key position): that key's score is made
    to stand out for that query (q and k share a large common direction), so that the output is that key's value if
    and only if the key is seen."""
    rng = np.random.default_rng(seed)
    q, k = rng.standard_normal((T, H, D)).astype(np.float32) * 0.3, rng.standard_normal((T, G, D)).astype(np.float32) * 0.3
    v = rng.standard_normal((T, G, V)).astype(np.float32)
    if loud:
        i, j = loud
        q[i, :, 0], k[j, :, 0] = 40.0, 40.0
    sink = rng.standard_normal(H).astype(np.float32)
    z = np.einsum("ihd,jhd->hij", q, np.repeat(k, H // G, axis=1)) * np.float32(scale)
    w = plain.softmax_with_sink(z, sink, plain.visible(T, window or T, keep))
    return q, k, v, sink, np.einsum("hij,jhv->ihv", w, np.repeat(v, H // G, axis=1)).reshape(T, H * V), w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_sink_window_and_kept_first_keys_in_prompts_and_decoding(dtype):
    """Keys just inside and just outside the window and the kept first keys, far keys, page borders: each made loud
    in turn; as a prompt from the step's rows and token by token from the paged cache (a ring behind pinned pages)."""
    from abacus_b200.cache import CacheNeed, SequenceCache
    from abacus_b200.kernels import ops
    from abacus_b200.parts import Workspace
    ws = Workspace(torch.device(DEV, torch.cuda.current_device()))
    H, G, D, V, window, keep, scale = 4, 2, 16, 24, 70, 5, 0.05
    T = 300  # five pages: the ring of three behind the pinned first page is gone round once
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    cases = [None, (299, 230), (299, 229), (299, 4), (299, 5), (150, 81), (150, 80), (133, 64), (133, 63), (129, 60),
             (75, 5), (75, 6), (72, 4), (69, 0), (200, 131), (200, 130), (270, 255), (260, 191), (260, 190), (257, 3)]
    for n_case, loud in enumerate(cases):
        q, k, v, sink, want, w = _attention_case(T, H, G, D, V, window, keep, scale, loud, seed=n_case)
        if dtype == torch.bfloat16:
            q, k, v = plain.bf16_round(q), plain.bf16_round(k), plain.bf16_round(v)
            z = np.einsum("ihd,jhd->hij", q, np.repeat(k, H // G, axis=1)) * np.float32(scale)
            w = plain.softmax_with_sink(z, sink, plain.visible(T, window, keep))
            want = np.einsum("hij,jhv->ihv", w, np.repeat(v, H // G, axis=1)).reshape(T, H * V)
        if loud:  # the loud key takes nearly all the weight exactly when it is seen
            i, j = loud
            seen = i - j < window or j < keep
            assert (w[:, i, j].min() > 0.9) == seen and (seen or w[:, i, j].max() == 0.0)
        row = np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1)
        need = CacheNeed(n_kv_heads=G, head_dim=D, window=window, v_head_dim=V, keep_first=keep)
        cache = SequenceCache([need], [None], 64 * 12, dtype, DEV, max_slots=4, max_context=64 * 12)
        kv = cache.views[0].kv
        assert kv.pinned_pages == 1 and kv.ring_pages == 3 and kv.table_width == 4
        cache.open_slot()  # slot 0 stays idle
        slot = cache.open_slot()
        # as a prompt: all rows at once, keys from the step
        cache.reserve(slot, T)
        b = batch_of([(slot, [0] * T, 0)])
        qkv = dev(row, dtype)
        out = torch.empty((T, H * V), dtype=dtype, device=DEV)
        ops.qkv_prep(qkv, H, G, D, b, None, None, None, None, None, 0, False, kv, v_dim=V)
        ops.attention_generic(qkv, out, H, G, D, scale, window, b, kv, from_step=True, v_dim=V, keep_first=keep, sink=dev(sink),
                              exact_weights=True)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, err_msg=f"prompt, loud {loud}", **tol)
        if dtype == torch.bfloat16:  # the same prompt on the tensor-core kernel
            fast = torch.empty_like(out)
            ops.attention_window(qkv, fast, H, G, D, scale, window, b, v_dim=V, keep_first=keep, sink=dev(sink))
            np.testing.assert_allclose(fast.float().cpu().numpy(), want, err_msg=f"prompt on tensor cores, loud {loud}", **tol)
        cache.advance(slot, T)
        # the prompt left its last window and its first keys in the cache: decode the last rows again from there
        if loud and loud[0] >= T - 5:
            for i in range(T - 5, T):
                b = batch_of([(slot, [0], i)])
                one = torch.empty((1, H * V), dtype=dtype, device=DEV)
                ops.attention_generic(dev(row[i:i + 1], dtype), one, H, G, D, scale, window, b, kv, v_dim=V, keep_first=keep,
                                      sink=dev(sink), exact_weights=True)
                np.testing.assert_allclose(one.float().cpu().numpy(), want[i:i + 1], err_msg=f"after the prompt, row {i}", **tol)
        cache.close_slot(slot)
        # token by token through the cache, in a slot that has just been used (its pages hold the other case's keys)
        if n_case % 3 == 0 or (loud and loud[0] < T - 5):
            slot = cache.open_slot()
            last = loud[0] if loud else T - 1
            for i in range(last + 1):
                cache.reserve(slot, i + 1)
                b = batch_of([(slot, [0], i)])
                qkv = dev(row[i:i + 1], dtype)
                ops.qkv_prep(qkv, H, G, D, b, None, None, None, None, None, 0, False, kv, v_dim=V)
                if i in (0, 1, 5, 63, 64, 69, 70, 71, 127, 128, 255, 256, last):
                    one = torch.empty((1, H * V), dtype=dtype, device=DEV)
                    ops.attention_generic(qkv, one, H, G, D, scale, window, b, kv, v_dim=V, keep_first=keep, sink=dev(sink),
                                          exact_weights=True)
                    np.testing.assert_allclose(one.float().cpu().numpy(), want[i:i + 1], err_msg=f"decoded row {i}, loud {loud}", **tol)
                    ops.attention_split(qkv, one, H, G, D, scale, window, b, kv, ws, v_dim=V, keep_first=keep, sink=dev(sink))
                    np.testing.assert_allclose(one.float().cpu().numpy(), want[i:i + 1], err_msg=f"decoded row {i} in parts, loud {loud}", **tol)
                cache.advance(slot, 1)
            cache.close_slot(slot)


@pytest.mark.parametrize("H,G,D,V,window,keep,with_sink", [(4, 2, 16, 24, 12, 3, True), (6, 2, 24, 40, 70, 0, True),
                                                          (3, 3, 32, 32, None, 0, False), (2, 2, 128, 128, 100, 7, True),
                                                          (1, 1, 256, 64, 5, 0, True), (2, 1, 40, 8, 64, 64, False),
                                                          (2, 1, 64, 128, 200, 130, True)])
def test_the_tensor_core_prompt_kernel_on_unequal_prompts(H, G, D, V, window, keep, with_sink):
    """Several sequences of unequal lengths in one step (one token, just under, at and just over a tile of 64 rows),
    every row against the plain formulas; head sizes that need padding to 16, windows shorter and longer than a tile."""
    from abacus_b200.kernels import ops
    lens, scale = [150, 1, 37, 64, 65, 300], 0.11
    rows, wants, sink = [], [], None
    for i, T in enumerate(lens):
        q, k, v, sk, _, _ = _attention_case(T, H, G, D, V, window, keep, scale, seed=100 + i)
        q, k, v = plain.bf16_round(q), plain.bf16_round(k), plain.bf16_round(v)
        sink = sk if sink is None else sink
        z = np.einsum("ihd,jhd->hij", q, np.repeat(k, H // G, axis=1)) * np.float32(scale)
        w = plain.softmax_with_sink(z, sink if with_sink else np.full(H, -np.inf, dtype=np.float32), plain.visible(T, window or T, keep))
        wants.append(np.einsum("hij,jhv->ihv", w, np.repeat(v, H // G, axis=1)).reshape(T, H * V))
        rows.append(np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1))
    b = batch_of([(i, [0] * T, 0) for i, T in enumerate(lens)])
    qkv = dev(np.concatenate(rows), torch.bfloat16)
    out = torch.empty((sum(lens), H * V), dtype=torch.bfloat16, device=DEV)
    assert ops.attention_window_takes(qkv, D, V, H, G)
    ops.attention_window(qkv, out, H, G, D, scale, window, b, v_dim=V, keep_first=keep, sink=dev(sink) if with_sink else None)
    got, want = out.float().cpu().numpy(), np.concatenate(wants)
    # float32 weights: what is left is the rounding of the stored result
    np.testing.assert_allclose(got, want, rtol=2 ** -8, atol=1e-3)


@pytest.mark.parametrize("H,G,D,V,window,keep,dtype", [(8, 1, 32, 200, None, 0, torch.bfloat16), (6, 2, 24, 40, 300, 9, torch.float32),
                                                        (16, 1, 64, 8, 130, 128, torch.bfloat16), (3, 3, 256, 130, 128, 0, torch.bfloat16)])
def test_decoding_in_parts_in_an_unequal_batch(H, G, D, V, window, keep, dtype):
    """Rows at very different positions in one decode step, each against the plain formulas: a first token, rows
    within one part of 128 keys, at its border, and over many parts; groups of up to 16 heads; values beyond 128."""
    from abacus_b200.cache import CacheNeed, SequenceCache
    from abacus_b200.kernels import ops
    from abacus_b200.parts import Workspace
    ws = Workspace(torch.device(DEV, torch.cuda.current_device()))
    lens, scale = [1, 500, 128, 129, 77], 0.2
    need = CacheNeed(n_kv_heads=G, head_dim=D, window=window, v_head_dim=V, keep_first=keep)
    cache = SequenceCache([need], [None], 64 * 32, dtype, DEV, max_slots=8, max_context=64 * 16)
    kv = cache.views[0].kv
    wants, last_rows, slots = [], [], []
    for i, T in enumerate(lens):
        q, k, v, sink, _, _ = _attention_case(T, H, G, D, V, window, keep, scale, seed=50 + i)
        if i == 0:
            sink0 = sink
        if dtype == torch.bfloat16:
            q, k, v = plain.bf16_round(q), plain.bf16_round(k), plain.bf16_round(v)
        z = np.einsum("ihd,jhd->hij", q, np.repeat(k, H // G, axis=1)) * np.float32(scale)
        w = plain.softmax_with_sink(z, sink0, plain.visible(T, window or T, keep))
        wants.append(np.einsum("hij,jhv->ihv", w, np.repeat(v, H // G, axis=1)).reshape(T, H * V)[-1])
        row = np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1)
        width = -(-row.shape[1] // 8) * 8
        row = np.concatenate([row, np.zeros((T, width - row.shape[1]), dtype=np.float32)], axis=1)
        slot = cache.open_slot()
        slots.append(slot)
        if T > 1:  # all but the last token as a prompt: its keys and values into the cache
            cache.reserve(slot, T - 1)
            b = batch_of([(slot, [0] * (T - 1), 0)])
            ops.qkv_prep(dev(row[:-1], dtype), H, G, D, b, None, None, None, None, None, 0, False, kv, v_dim=V, row=width)
            cache.advance(slot, T - 1)
        last_rows.append(row[-1])
    for slot, T in zip(slots, lens):
        cache.reserve(slot, T)
    b = batch_of([(slot, [0], T - 1) for slot, T in zip(slots, lens)])
    qkv = dev(np.stack(last_rows), dtype)
    ops.qkv_prep(qkv, H, G, D, b, None, None, None, None, None, 0, False, kv, v_dim=V, row=width)
    out = torch.empty((len(lens), H * V), dtype=dtype, device=DEV)
    ops.attention_split(qkv, out, H, G, D, scale, window, b, kv, ws, v_dim=V, keep_first=keep, sink=dev(sink0), row=width)
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=2 ** -8, atol=2e-3)
    np.testing.assert_allclose(out.float().cpu().numpy(), np.stack(wants), **tol)


def test_a_large_sink_takes_the_weight_and_no_sink_is_plain_softmax():
    from abacus_b200.kernels import ops
    H, G, D, V, T = 2, 1, 8, 8, 6
    q, k, v, sink, _, _ = _attention_case(T, H, G, D, V, None, 0, 0.3)
    row = np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1)
    b = batch_of([(0, [0] * T, 0)])
    z = np.einsum("ihd,jhd->hij", q, np.repeat(k, H, axis=1)) * np.float32(0.3)
    for s in (np.array([30.0, -30.0], dtype=np.float32), None):
        w = plain.softmax_with_sink(z, s if s is not None else np.full(H, -np.inf, dtype=np.float32), plain.visible(T, T, 0))
        want = np.einsum("hij,jhv->ihv", w, np.repeat(v, H, axis=1)).reshape(T, H * V)
        out = torch.empty((T, H * V), dtype=torch.float32, device=DEV)
        ops.attention_generic(dev(row), out, H, G, D, 0.3, None, b, None, from_step=True, v_dim=V,
                              sink=dev(s) if s is not None else None, exact_weights=True)
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-4, atol=1e-5)
        if s is not None:
            assert np.abs(want[:, :V]).max() < 1e-6 < np.abs(want[:, V:]).max()  # head 0 gives its weight to the sink


# ------------------------------------------------------------------ whole models through the engine
def _engine(tmp_path, name, dtype, **kw):
    from abacus_b200.engine import Engine, load_model
    folder, raw, tensors = tm.write_folder(tmp_path, name)
    model = load_model(folder, dtype)
    return Engine(model, **{"max_tokens": 64 * 24, **kw}), raw, tensors, folder


def _oracle(raw, tensors, tokens, dtype):
    """(plain logits in the engine's manner, the noise to allow for)."""
    if dtype == "float32":
        want = plain.forward(raw, tensors, tokens)
        return want, float(np.abs(want - plain.forward(raw, tensors, tokens, real=np.float64)).max())
    want = plain.forward(raw, tensors, tokens, rnd=plain.bf16_round)
    return want, float(np.abs(want - plain.forward(raw, tensors, tokens)).max())


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "float32"), ("R", "float32"), ("S", "float32"),
                                        ("Q", "bfloat16"), ("R", "bfloat16"), ("S", "bfloat16")])
def test_prompts_decoding_batches_and_used_slots_against_the_plain_model(tmp_path, name, dtype):
    engine, raw, tensors, _ = _engine(tmp_path, name, dtype)
    rng = np.random.default_rng(7)
    vocab = raw["vocab"]
    lens = [150, 1, 37, 80]
    seqs = [[int(t) for t in rng.integers(0, vocab, n)] for n in lens]
    oracle = [_oracle(raw, tensors, s, dtype) for s in seqs]
    # each alone, whole, all logits wanted; the slot is given back and used again by the next
    for s, (want, noise) in zip(seqs, oracle):
        slot = engine.open()
        got = engine.step([(slot, s, list(range(len(s))))]).cpu().numpy()
        engine.close(slot)
        assert_logits(got, want, dtype, f"{name} whole, {len(s)} tokens", noise)
    # together in one batch of unequal prompts, cut before their ends, then decoded together; early enders leave
    cut = [100, 1, 20, 64]
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


@pytest.mark.parametrize("name", ["P", "R"])
def test_token_by_token_from_the_first_token_and_long_decoding(tmp_path, name):
    """No prompt at all: every token a step of its own, past the window, the kept keys and three pages."""
    engine, raw, tensors, _ = _engine(tmp_path, name, "float32")
    rng = np.random.default_rng(3)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 200)]
    want, noise = _oracle(raw, tensors, tokens, "float32")
    slot = engine.open()
    got = np.concatenate([engine.step([(slot, [t], [0])]).cpu().numpy() for t in tokens])
    engine.close(slot)
    assert_logits(got, want, "float32", f"{name} token by token", noise)


def test_graphs_and_plain_launches_give_the_same_bits_and_states_survive_a_capture(tmp_path):
    from abacus_b200.engine import Engine
    engine, raw, tensors, _ = _engine(tmp_path, "P", "float32")
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
    folder, raw, tensors = tm.write_folder(tmp_path, "P")
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
    folder, raw, tensors = tm.write_folder(tmp_path, "R")
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
