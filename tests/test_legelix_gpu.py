"""Legelix in the engine against the plain implementation (tests/plain_legelix.py): each kernel of its
mechanisms alone, then whole models under every way of cutting the work, in 32-bit and in bfloat16:
whole prompts, long decoding one token at a time across several chunk edges, portions down to two
tokens (and single first tokens), mixed batches of unequal requests with so few pages and state slots
that both are used again (pages given back are filled with NaN), and greedy generation through the
engine's own entry point and scheduler.  Where random weights would hide a fault (a key far back, the
edge of a chunk, a sink), inputs are made so that it shows."""

import functools
import json

import numpy as np
import pytest
import torch

from legelix_models import CONFIGS, DECAY_RANK, PAGE_SIZE, read_model, write_model
from plain_legelix import (F64, plain_attention_core, plain_layer_norm, plain_legelix, plain_rotary_frequencies,
                           plain_rotate, plain_unit_rms, silu, softplus)
from replay_util import (collect, peak_tokens, random_tokens, tolerance, trace_batched_tail, trace_mixed,
                         trace_portions, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, dtype: str):
        if (name, dtype) not in made:
            made[(name, dtype)] = write_model(tmp_path_factory.mktemp(f"legelix_{name}_{dtype}"), CONFIGS[name],
                                              DECAY_RANK[name], seed=17 + ord(name), dtype=DTYPES[dtype])
        return made[(name, dtype)]

    return get


@functools.lru_cache(maxsize=128)
def _plain(folder: str, tokens: tuple) -> np.ndarray:
    config, weights = read_model(folder)
    return plain_legelix(config, weights, list(tokens))[0].numpy()


def replay(folder, dtype, steps, page_size, max_requests=4, graphs=True):
    from zephyr_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(folder, dtype, peak_tokens(steps, max(64, page_size)), page_size=page_size,
                             max_requests=max_requests)
    replayer.runner.poison_freed_pages = True
    replayer.runner.use_cuda_graphs = graphs
    outputs = {}
    for step in steps:
        result = replayer.step(step)
        if result is not None:
            outputs[step["step"]] = result
        replayer.runner.manager.check_invariants()
    return outputs


def assert_rows_match(rows, requests, folder, dtype, what):
    """Every row of logits within its bound (``replay_util.tolerance``).  In bfloat16 a layer norm that
    follows a part's output magnifies the rounding of that output wherever the output's spread over
    the width happens to be small, so single positions lie a few times further out than the rest
    (measured: mean 0.3 of the bound, one position in a hundred at 1 to 4 bounds); there the rule
    is: no row beyond six bounds, and no more than one row in twenty-five beyond one (the float32 run's
    error rises at the same positions: they are badly conditioned, not wrongly computed).  A fault of a mask, a
    state or a page moves logits by hundreds of bounds.  In float32 every row is within its bound."""
    ratios = {}
    for (rid, position), got in sorted(rows.items()):
        expected = _plain(str(folder), tuple(requests[rid]))[position]
        assert np.isfinite(got).all(), f"{what}: non-finite logits for {rid} at {position}"
        ratios[(rid, position)] = float(np.abs(got.astype(np.float64) - expected).max()) / tolerance(dtype, expected)
    over = [key for key, ratio in ratios.items() if ratio > 1.0]
    worst = max(ratios, key=ratios.get)
    print(f"[legelix] {what} {dtype}: worst error {ratios[worst]:.2f} of its bound at {worst}, {len(over)} of {len(ratios)} beyond it")
    limit, allowed = (1.0, 0) if dtype == "float32" else (6.0, max(1, len(ratios) // 25))
    assert ratios[worst] <= limit and len(over) <= allowed, \
        f"{what}: first wrong logits at request {over[0][0]} position {over[0][1]}: {ratios[over[0]]:.2f} bounds"


LENGTHS = {"P": [70, 128, 45, 33, 100, 5, 17, 64], "Q": [1, 9, 33, 70, 41, 96, 23, 2], "R": [150, 40, 66, 129, 31, 200],
           "S": [170, 40, 81, 129, 31, 300, 72, 5]}
TRACES = {"whole": trace_whole, "tail": functools.partial(trace_tail, tail=60),
          "portions": functools.partial(trace_portions, sizes=(1, 1, 2, 7, 2, 5, 3, 2, 11, 2, 4, 1, 6, 23)),
          "mixed": trace_mixed, "batched": trace_batched_tail}


def make_requests(name):
    return {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, seed=100 * ord(name) + i)
            for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("mode", list(TRACES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_replay_matches_plain(folders, cuda_device, name, dtype, mode):
    folder, requests = folders(name, dtype), make_requests(name)
    steps = TRACES[mode](requests)
    rows = collect(steps, replay(folder, dtype, steps, PAGE_SIZE[name]))
    assert_rows_match(rows, requests, folder, dtype, f"{name} {mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_state_slots_are_used_again_and_again(folders, cuda_device, dtype):
    """Eight requests through two slots: a state that a new request inherits would show at its first token."""
    folder, requests = folders("P", dtype), make_requests("P")
    steps = trace_mixed(requests, max_live=2, seed=5)
    rows = collect(steps, replay(folder, dtype, steps, PAGE_SIZE["P"], max_requests=2))
    assert_rows_match(rows, requests, folder, dtype, "P two slots")


def test_captured_steps_equal_launched_ones(folders, cuda_device):
    """Steps replayed from CUDA graphs (a step that is run once to warm up and once for real must not
    advance a state twice) give the logits of steps launched kernel by kernel."""
    folder, requests = folders("P", "float32"), make_requests("P")
    steps = trace_batched_tail(requests, tail=20)
    with_graphs = collect(steps, replay(folder, "float32", steps, 16, graphs=True))
    without = collect(steps, replay(folder, "float32", steps, 16, graphs=False))
    for key, row in without.items():
        assert np.array_equal(row, with_graphs[key]), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_chunk_edges(folders, cuda_device, dtype):
    """A short prompt and 190 tokens decoded one by one: 19 chunk edges of Q, 7 of P."""
    for name in ("Q", "P", "S"):
        folder = folders(name, dtype)
        requests = {"long": random_tokens(CONFIGS[name]["vocab"], 200, seed=9)}
        steps = trace_tail(requests, tail=190)
        assert_rows_match(collect(steps, replay(folder, dtype, steps, PAGE_SIZE[name])), requests, folder, dtype,
                          f"{name} long decoding")


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("P", "bfloat16"), ("Q", "float32"), ("R", "bfloat16")])
def test_greedy_generation_through_the_engine(folders, cuda_device, name, dtype):
    from zephyr_b200 import Engine
    from zephyr_b200.engine import KvCacheOptions, PagedSchedulerConfig

    folder = folders(name, dtype)
    config, weights = read_model(folder)
    engine = Engine(folder, dtype=dtype, max_seq_len=256,
                    scheduler=PagedSchedulerConfig(max_num_seqs=3, max_num_batched_tokens=16, max_prefill_chunk_tokens=7),
                    kv_cache=KvCacheOptions(block_size=PAGE_SIZE[name], num_blocks=40))
    prompts = [random_tokens(config["vocab"], n, seed=n) for n in (5, 11, 17, 40, 3)]
    outputs = engine.generate(prompts, max_tokens=10, temperature=0.0, ignore_eos=True)
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for index, got in enumerate(output.token_ids):
            logits = plain_legelix(config, weights, tokens)[0][-1]
            top = torch.topk(logits, 2).values
            if got != int(logits.argmax()):
                # a first difference is forgiven where the two best lie closer than twice the engine's bound
                assert float(top[0] - top[1]) <= 2 * tolerance(dtype, logits.numpy()), (prompt, index)
                break
            tokens.append(got)
        assert output.usage.completion_tokens == 10
    assert engine.runner.manager.num_requests == 0
    engine.runner.manager.check_invariants()


def test_the_replay_program_on_legelix(folders, cuda_device, tmp_path):
    """bin/trace_run picks the architecture from config.json and writes the logits of a mixed trace."""
    import subprocess
    import sys
    from pathlib import Path

    folder, requests = folders("Q", "float32"), make_requests("Q")
    steps = trace_mixed(requests, seed=3)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(peak_tokens(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, CONFIGS["Q"]["vocab"])
               for s in steps if any(e["want"] for e in s["entries"])}
    assert_rows_match(collect(steps, outputs), requests, folder, "float32", "Q through the program")


# ------------------------------------------------------------------------------------- kernels alone
def _rows(lengths, device):
    starts = np.concatenate([[0], np.cumsum(lengths[:-1])]).astype(np.int32)
    return (torch.tensor(starts, dtype=torch.int32, device=device),
            torch.tensor(lengths, dtype=torch.int32, device=device))


@pytest.mark.parametrize("width", [48, 257, 1024, 5000])
def test_layer_norm_and_the_fused_residual_form(cuda_device, width):
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3 + 0.5
    delta = torch.randn(7, width, generator=g)
    w1, b1, w2, b2 = (torch.randn(width, generator=g) for _ in range(4))
    dev = lambda t: t.to(cuda_device)
    expected = plain_layer_norm(x.double(), w1.double(), b1.double(), 1e-5)
    got = ops.layer_norm(dev(x), dev(w1), dev(b1), 1e-5)
    assert (got.cpu().double() - expected).abs().max() < 2e-5
    got16 = ops.layer_norm(dev(x), dev(w1), dev(b1), 1e-5, out_dtype=torch.bfloat16)
    assert got16.dtype == torch.bfloat16 and (got16.cpu().double() - expected).abs().max() < 0.05
    for dtype, bound in ((torch.float32, 3e-5), (torch.bfloat16, 0.06)):
        residual = dev(x.clone())
        d = dev(delta.to(dtype))
        out = ops.residual_layer_norm(residual, d, dev(w1), dev(b1), 1e-5, 0.3, dev(w2), dev(b2), 1e-6)
        summed = x.double() + 0.3 * plain_layer_norm(d.cpu().double(), w1.double(), b1.double(), 1e-5)
        assert (residual.cpu().double() - summed).abs().max() < 3e-5          # the stream stays float32
        assert out.dtype == dtype
        assert (out.cpu().double() - plain_layer_norm(summed, w2.double(), b2.double(), 1e-6)).abs().max() < bound
        alone = dev(x.clone())
        assert ops.residual_layer_norm(alone, d, dev(w1), dev(b1), 1e-5, 0.3) is None
        assert torch.equal(alone, residual)


@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 24), (1, 144, 40), (3, 256, 8), (4, 32, 33)])
def test_gated_recurrence_and_its_state(cuda_device, heads, dim, vdim):
    """The scan over rows of unequal length, in portions, from and to slots; decays close to one keep a
    token from far back alive, so a state lost between two portions shows."""
    from zephyr_b200.kernels import ops

    g = torch.Generator().manual_seed(dim)
    lengths, slots = [37, 1, 9], [2, 0, 3]
    T = sum(lengths)
    dev = lambda t: t.to(cuda_device)
    q, k, v = (torch.randn(T, heads * n, generator=g) for n in (dim, dim, vdim))
    z = torch.randn(T, heads * dim, generator=g) + 4.0
    bias = torch.randn(heads * dim, generator=g) * 0.5
    tau, scale = 4.0, dim ** -0.5
    state = torch.zeros(4, heads * dim * vdim, device=cuda_device)
    state[1] = float("nan")                          # a slot nobody uses is not touched
    status = ops.new_status(cuda_device)

    def plain(rows_q, rows_k, rows_v, rows_z, S):
        out = []
        for t in range(rows_q.shape[0]):
            a = torch.exp(torch.nn.functional.logsigmoid(rows_z[t].double() + bias.double()) / tau).view(heads, dim)
            S = a[:, :, None] * S + rows_k[t].double().view(heads, dim)[:, :, None] * rows_v[t].double().view(heads, vdim)[:, None, :]
            out.append(torch.einsum("hdv,hd->hv", S, rows_q[t].double().view(heads, dim) * scale).reshape(-1))
        return torch.stack(out), S

    # two steps: the first portions, then the rest
    first = [20, 1, 4]
    expected, got = [None] * 3, [None] * 3
    S_plain = [torch.zeros(heads, dim, vdim, dtype=F64) for _ in lengths]
    offsets = np.concatenate([[0], np.cumsum(lengths)])
    for step in range(2):
        spans = []
        for r, n in enumerate(lengths):
            lo = offsets[r] + (0 if step == 0 else first[r])
            hi = offsets[r] + (first[r] if step == 0 else n)
            spans.append((r, int(lo), int(hi)))
        spans = [s for s in spans if s[2] > s[1]]
        index = torch.cat([torch.arange(lo, hi) for _, lo, hi in spans])
        starts, lens = _rows([hi - lo for _, lo, hi in spans], cuda_device)
        o = ops.decayed_state_scan("gated", dev(q[index]), dev(k[index]), dev(v[index]), heads, dim, vdim, state,
                                   torch.tensor([slots[r] for r, _, _ in spans], dtype=torch.int32, device=cuda_device),
                                   starts, lens, status, decay_logits=dev(z[index]), decay_bias=dev(bias),
                                   inv_tau=1.0 / tau, q_scale=scale).cpu().double()
        at = 0
        for r, lo, hi in spans:
            want, S_plain[r] = plain(q[lo:hi], k[lo:hi], v[lo:hi], z[lo:hi], S_plain[r])
            assert (o[at:at + hi - lo] - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max())), (step, r)
            at += hi - lo
    ops.check_status(status)
    for r, slot in enumerate(slots):
        assert (state[slot].cpu().double().view(heads, dim, vdim) - S_plain[r]).abs().max() < 2e-4 * max(1.0, float(S_plain[r].abs().max()))
    assert torch.isnan(state[1]).all()


@pytest.mark.parametrize("mode", ["gated", "state_space"])
def test_long_rows_in_segments_equal_rows_in_one_piece(cuda_device, mode):
    """Requests of 700, 40 and 300 tokens in segments of 64 that run side by side (a pass from zero, the
    carry, a pass with outputs) against the same step token by token in one piece: outputs and final
    states agree to rounding, from states that are not zero."""
    from zephyr_b200.kernels import ops

    heads, dim, vdim, groups = 4, 48, 40, 2
    g = torch.Generator().manual_seed(11)
    lengths = [700, 40, 300]
    T = sum(lengths)
    starts, lens = _rows(lengths, cuda_device)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=cuda_device)
    dev = lambda t: t.to(cuda_device)
    start_state = torch.randn(3, heads * dim * vdim, generator=g)
    status = ops.new_status(cuda_device)
    if mode == "gated":
        q, k, v = (dev(torch.randn(T, heads * n, generator=g)) for n in (dim, dim, vdim))
        z, bias = torch.randn(T, heads * dim, generator=g) + 3.0, dev(torch.randn(heads * dim, generator=g))
        run = lambda state, segment: ops.decayed_state_scan(
            "gated", q, k, v, heads, dim, vdim, state, slots, starts, lens, status, decay_logits=dev(z.clone()),
            decay_bias=bias, inv_tau=0.25, q_scale=0.1, segment=segment)
    else:
        q, k = (dev(torch.randn(T, groups * dim, generator=g)) for _ in range(2))
        v, dt = dev(torch.randn(T, heads * vdim, generator=g)), dev(torch.randn(T, heads, generator=g) - 2.0)
        consts = [dev(torch.randn(heads, generator=g) * 0.5) for _ in range(3)]
        run = lambda state, segment: ops.decayed_state_scan(
            "state_space", q, k, v, heads, dim, vdim, state, slots, starts, lens, status, dt=dt, dt_bias=consts[0],
            a_log=consts[1], skip=consts[2], heads_per_group=heads // groups, segment=segment)
    whole_state, cut_state = dev(start_state.clone()), dev(start_state.clone())
    whole, cut = run(whole_state, 0), run(cut_state, 64)
    ops.check_status(status)
    scale = float(whole.abs().max())
    assert (whole - cut).abs().max().item() < 2e-5 * scale
    assert (whole_state - cut_state).abs().max().item() < 2e-5 * float(whole_state.abs().max())
    assert not torch.equal(whole_state.cpu(), start_state)


def test_state_space_recurrence_convolution_and_gated_norm(cuda_device):
    """The Mamba-2 path after its input projection, kernel by kernel against the equations: a row cut
    in two (the convolution's last inputs and the state carried in the slot) beside a whole one."""
    from zephyr_b200.kernels import ops

    heads, vdim, N, groups, taps, parts = 6, 20, 24, 3, 4, 2
    inner, gn = heads * vdim, groups * N
    channels = inner + 2 * gn
    g = torch.Generator().manual_seed(4)
    T = 29
    projected = torch.randn(T, 2 * inner + 2 * gn + heads, generator=g)
    conv_w, conv_b = torch.randn(channels, taps, generator=g) * 0.5, torch.randn(channels, generator=g) * 0.2
    dt_bias, a_log, skip = (torch.randn(heads, generator=g) for _ in range(3))
    norm_w = torch.randn(inner, generator=g)
    dev = lambda t: t.to(cuda_device)

    # the equations
    P = projected.double()
    zg, xbc, dt = P[:, :inner], P[:, inner:inner + channels], P[:, inner + channels:]
    padded = torch.cat([torch.zeros(taps - 1, channels, dtype=F64), xbc])
    mixed = silu(sum(padded[j:j + T] * conv_w.double()[:, j] for j in range(taps)) + conv_b.double())
    x, B, C = mixed[:, :inner].view(T, heads, vdim), mixed[:, inner:inner + gn].view(T, groups, N), mixed[:, inner + gn:].view(T, groups, N)
    step = softplus(dt + dt_bias.double())
    S, ys = torch.zeros(heads, N, vdim, dtype=F64), []
    of = [h // (heads // groups) for h in range(heads)]
    for t in range(T):
        S = torch.exp(-torch.exp(a_log.double()) * step[t])[:, None, None] * S + step[t][:, None, None] * B[t][of][:, :, None] * x[t][:, None, :]
        ys.append(torch.einsum("hnp,hn->hp", S, C[t][of]) + skip.double()[:, None] * x[t])
    y = torch.stack(ys).reshape(T, inner)
    expected = plain_unit_rms((y * silu(zg)).view(T, parts, inner // parts), 1e-5).reshape(T, inner) * norm_w.double()

    scan = heads * N * vdim
    store = torch.zeros(3, scan + (taps - 1) * channels, device=cuda_device)
    status = ops.new_status(cuda_device)
    results = {}
    for slot, cuts in ((1, [T]), (2, [11, 2, 16])):
        outs, at = [], 0
        for n in cuts:
            part = dev(projected[at:at + n].contiguous())
            starts, lens = _rows([n], cuda_device)
            slots = torch.tensor([slot], dtype=torch.int32, device=cuda_device)
            m = ops.causal_conv_silu(part[:, inner:], channels, dev(conv_w), dev(conv_b), store[:, scan:], slots, starts,
                                     lens, torch.zeros(n, dtype=torch.int32, device=cuda_device), status)
            assert (m.cpu().double() - mixed[at:at + n]).abs().max() < 1e-5
            o = ops.decayed_state_scan("state_space", m[:, inner + gn:], m[:, inner:inner + gn], m[:, :inner], heads, N,
                                       vdim, store[:, :scan], slots, starts, lens, status, dt=part[:, inner + channels:],
                                       dt_bias=dev(dt_bias), a_log=dev(a_log), skip=dev(skip),
                                       heads_per_group=heads // groups)
            outs.append(ops.gated_group_rms_norm(o, part[:, :inner], dev(norm_w), inner // parts, 1e-5, gate_first=True))
            at += n
        results[slot] = torch.cat(outs).cpu().double()
        assert (results[slot] - expected).abs().max() < 2e-4 * float(expected.abs().max())
    ops.check_status(status)
    assert (store[1] - store[2]).abs().max() < 1e-5 and store[0].abs().max() == 0
    # the other order of gate and norm, one scale vector shared by the groups
    o = torch.randn(5, 48, generator=g)
    gate, w = torch.randn(5, 48, generator=g), torch.randn(16, generator=g)
    got = ops.gated_group_rms_norm(dev(o), dev(gate), dev(w), 16, 1e-6, gate_first=False).cpu().double()
    want = (plain_unit_rms(o.double().view(5, 3, 16), 1e-6) * w.double()).reshape(5, 48) * silu(gate.double())
    assert (got - want).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kd,vd,heads,kv_heads,chunk,rot_dims,page", [(32, 16, 4, 2, 24, 16, 16), (24, 40, 3, 3, 10, 24, 16),
                                                                   (64, 64, 8, 1, 200, 32, 32), (18, 6, 2, 1, 0, 0, 16),
                                                                   (32, 16, 4, 2, 24, 0, 16), (16, 48, 2, 2, 16, 0, 32),
                                                                   (32, 32, 4, 2, 40, 0, 16), (128, 128, 4, 1, 100, 64, 16),
                                                                   (96, 96, 6, 2, 33, 0, 32)])
def test_chunked_sink_attention_at_its_edges(cuda_device, dtype, kd, vd, heads, kv_heads, chunk, rot_dims, page):
    """Queries that point at one key each: the key far back in the chunk, the first key of the chunk, and
    the last key of the chunk before (which must not be seen), in a prompt's portion and decoded
    alone, over pages that are not in order; and a sink that takes most of the weight on one head."""
    from zephyr_b200.kernels import ops

    torch_dtype = DTYPES[dtype]
    g = torch.Generator().manual_seed(kd + vd)
    T = 3 * (chunk or 40) + 7
    size = chunk or None
    q = torch.randn(T, heads, kd, generator=g)
    k = torch.randn(T, kv_heads, kd, generator=g)
    v = torch.randn(T, kv_heads, vd, generator=g)
    group = heads // kv_heads
    # position p of head 0 looks for the key at: the start of its chunk, the end of the chunk before, far back
    targets = {}
    for p in range(T - 30, T):
        start = (p // chunk) * chunk if chunk else 0
        target = (start, start - 1, max(start, p - (chunk or 40) + 2))[p % 3]
        if target < 0:
            continue
        targets[p] = target
    for target in set(targets.values()):
        k[target, 0] *= 4.0                        # a long key, so that the match below beats every chance alignment
    for p, target in targets.items():
        q[p, 0] = k[target, 0] * 2.0               # a score of 32 |k|^2 against about 8 |k| |k'| cos for the rest
    sinks = torch.randn(heads, generator=g)
    sinks[-1] = 80.0                            # the last head gives nearly everything to its sink
    freqs = plain_rotary_frequencies({"base": 100.0, "dims": rot_dims}) if rot_dims else None
    positions = torch.arange(T)
    bias = torch.randn(heads * kd + kv_heads * (kd + vd), generator=g) * 0.1
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1)
    # the plain side: bias, then rotation (no norm here), then the chunked softmax with the sink
    full = qkv.double() + bias.double()
    pq = full[:, :heads * kd].view(T, heads, kd)
    pk = full[:, heads * kd:heads * kd + kv_heads * kd].view(T, kv_heads, kd)
    pv = full[:, heads * kd + kv_heads * kd:].view(T, kv_heads, vd)
    if rot_dims:
        pq, pk = plain_rotate(pq, positions, freqs, rot_dims), plain_rotate(pk, positions, freqs, rot_dims)
    scale = 1.0 / 3.0 if rot_dims == 0 else 0.11
    expected = plain_attention_core(pq, pk, pv, scale, size, sinks.double()).reshape(T, heads * vd)

    blocks = -(-T // page)
    order = torch.randperm(blocks, generator=g) + 1         # pages out of order; page 0 is the null page
    table = order.to(torch.int32).view(1, -1).to(cuda_device)
    cache = torch.full((blocks + 1, kv_heads * page * (kd + vd)), float("nan"), dtype=torch_dtype, device=cuda_device)
    status = ops.new_status(cuda_device)
    tile = ops.attention_tile_tokens(group)
    outs, at = [], 0
    cuts = [T - 12] + [1] * 12                              # a portion, then twelve tokens alone
    for n in cuts:
        rows = (torch.tensor([0], dtype=torch.int32, device=cuda_device), torch.tensor([n], dtype=torch.int32, device=cuda_device),
                torch.tensor([at], dtype=torch.int32, device=cuda_device))
        pos = torch.arange(at, at + n, dtype=torch.int32, device=cuda_device)
        qs = ops.qkv_pairs(qkv[at:at + n].to(cuda_device), heads, kv_heads, kd, vd, bias.to(cuda_device), None, None, 0.0,
                           freqs.float().to(cuda_device) if rot_dims else None, rot_dims, pos,
                           torch.zeros(n, dtype=torch.int32, device=cuda_device), cache, table, status, torch_dtype)
        tile_q0 = torch.arange(0, n, tile, dtype=torch.int32, device=cuda_device)
        outs.append(ops.paged_attention(qs, cache, table, torch.zeros_like(tile_q0), tile_q0, tile, *rows, heads, kv_heads,
                                        kd, 0, scale, status, value_dim=vd, chunk=chunk, sinks=sinks.to(cuda_device)))
        if kd == vd and ops.paged_decode_supported(heads, kv_heads, kd, torch_dtype):
            # the same tokens through the kernels for prompts and for single tokens: they mask and count alike
            paged = cache.view(blocks + 1, 2, kv_heads, page, kd)
            fast = torch.full_like(outs[-1], float("nan"))
            if n == 1:
                ops.paged_decode(qs, paged, table, rows[0], rows[0], rows[2], at + 1, heads, kv_heads, kd, 0, scale,
                                 status, fast, chunk=chunk, sinks=sinks.to(cuda_device))
            else:
                wide = ops.paged_prefill_tile_tokens()
                wide_q0 = torch.arange(0, n, wide, dtype=torch.int32, device=cuda_device)
                ops.paged_prefill(qs, paged, table, torch.zeros_like(wide_q0), wide_q0, *rows, heads, kv_heads, kd, 0,
                                  scale, status, fast, chunk=chunk, sinks=sinks.to(cuda_device))
            assert (fast.double() - outs[-1].double()).abs().max().item() < 0.03 * max(1.0, float(expected.abs().max())), (n, at)
        at += n
    ops.check_status(status)
    got = torch.cat(outs).cpu().double()
    assert torch.isfinite(got).all()
    bound = 2e-5 if dtype == "float32" else 0.04
    assert (got - expected).abs().max() < bound * max(1.0, float(expected.abs().max()))
    # what the test is for: the pointed-at key decides head 0's output when it is inside the chunk
    if dtype == "float32" and rot_dims == 0:
        for p, target in targets.items():
            start = (p // chunk) * chunk if chunk else 0
            close = (got[p, :vd] - pv[target, 0]).abs().max() < 0.2
            assert bool(close) == (target >= start), (p, target)
    assert got[:, (heads - 1) * vd:].abs().max() < 1e-6       # the sink's head has given nearly all weight away
