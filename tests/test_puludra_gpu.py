"""Puludra through the engine against the plain implementation.

Replays through bin/trace_run: the same requests whole, with their last tokens one by one, in
portions of changing size down to two tokens, and mixed (up to four live, portions beside single
tokens, few pages and four state slots so that both are used again, freed pages filled with NaN),
in float32 and bfloat16, also from captured CUDA graphs.  "Sharp" variants scale queries and move
gate bounds so that a lost far key, a key leaked from the future or a lost state shows.
Generation through LLMEngine and ContinuousBatchingEngine.  The kernels one by one."""
import math

import pytest
import torch

import plain_puludra as plain
import puludra_util as pu
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [1, 9, 40, 131, 260], "odd": [2, 17, 64, 150], "wide": [3, 33, 97, 200],
           "only_latent": [1, 15, 16, 17, 70], "only_hgrn2": [1, 2, 45, 100], "only_retention": [1, 31, 90]}


def replay(name, dtype, tmp_path, cuda_graph=False, sharp=False):
    spec = pu.CONFIGS[name]
    model_dir = str(tmp_path / "model")
    config, weights = pu.make_folder(model_dir, name, sharp=sharp)
    prompts = {f"p{n}": ru.random_ids(n, config["vocab"], 100 + n) for n in LENGTHS[name]}
    trace, peak = ru.build_four_mode_trace(prompts, spec["page_size"])
    got = ru.run_trace(model_dir, dtype, trace, peak, str(tmp_path / "out"), page_size=spec["page_size"],
                       cuda_graph=cuda_graph, max_requests=4)
    refs = {n: plain.forward(weights, config, ids).float() for n, ids in prompts.items()}
    modes = set()
    for (step, rid, pos), row in got.items():
        mode, pname = rid.split("/")
        modes.add(mode.rstrip("01"))
        ref = refs[pname][pos]
        assert torch.isfinite(row).all(), (step, rid, pos)
        err = (row - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1e-3)
        if dtype == "float32":
            assert err <= 2e-4 * max(scale, 1.0), f"first wrong place: step {step} request {rid} position {pos}: {err}"
        else:
            assert err <= 0.03 * scale + 0.02, f"first wrong place: step {step} request {rid} position {pos}: {err}"
    assert modes == {"whole", "tail", "portions", "mixed"}


@pytest.mark.parametrize("name", sorted(pu.CONFIGS))
def test_replay_float32(name, tmp_path):
    replay(name, "float32", tmp_path)


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_replay_bfloat16(name, tmp_path):
    replay(name, "bfloat16", tmp_path)


@pytest.mark.parametrize("name", ["mix", "wide"])
def test_replay_bfloat16_single_token_steps_from_captured_graphs(name, tmp_path):
    replay(name, "bfloat16", tmp_path, cuda_graph=True)


@pytest.mark.parametrize("name", ["mix", "only_latent", "only_hgrn2"])
def test_replay_float32_sharp_far_keys_and_long_memories(name, tmp_path):
    replay(name, "float32", tmp_path, sharp=True)


def test_sharpening_makes_far_tokens_matter():
    """The sharp weights do what they are for: cutting the first tokens off changes late logits."""
    config = pu.CONFIGS["mix"]["config"]
    w = pu.sharpen(config, plain.random_weights(config, pu.CONFIGS["mix"]["seed"]))
    ids = ru.random_ids(150, config["vocab"], 5)
    a = plain.forward(w, config, ids)[-1]
    b = plain.forward(w, config, ids[8:])[-1]
    assert (a - b).abs().max() > 0.05


# ------------------------------------------------------------------ generation entry points
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("mix", "wide"):
        d = str(tmp_path_factory.mktemp(f"puludra_{name}"))
        out[name] = (d,) + pu.make_folder(d, name)
    return out


def load(folder, dtype):
    from dispec_b200 import load_model
    return load_model(folder, dtype, "cuda:0")


def assert_greedy(weights, config, prompt, got, dtype):
    """Teacher-forced on the engine's tokens: each equals the plain argmax, or the plain top-2 gap
    there is below what the type can resolve."""
    logits = plain.forward(weights, config, list(prompt) + list(got)).float()
    for i, tok in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        top2 = torch.topk(row, 2)
        reach = 1e-4 if dtype == "float32" else 2 * (0.03 * row.abs().max().item() + 0.02)
        assert tok == int(top2.indices[0]) or float(top2.values[0] - top2.values[1]) < reach, (i, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_llm_engine(folders, dtype):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["mix"]
    engine = LLMEngine(load(folder, dtype), num_blocks=32, cuda_graph=dtype == "bfloat16")
    for n in (1, 9, 40):  # the same engine: pages and the state slot are used again
        prompt = ru.random_ids(n, config["vocab"], 300 + n)
        got = engine.generate(prompt, 10, SamplingParams(temperature=0.0))
        assert len(got) == 10
        assert_greedy(weights, config, prompt, got, dtype)
    assert engine.runner.cache.num_free_pages() == 32 and engine.runner.cache.free_slots() == 4


def test_long_decoding_float32(folders):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["mix"]
    engine = LLMEngine(load(folder, "float32"), num_blocks=32)
    prompt = ru.random_ids(3, config["vocab"], 1)
    got = engine.generate(prompt, 200, SamplingParams())
    assert len(got) == 200
    assert_greedy(weights, config, prompt, got, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_continuous_batching_more_requests_than_slots(folders, dtype):
    """Seven requests through three state slots and a small pool: portions of prompts beside
    decoded tokens; slots and pages of finished requests go to waiting ones."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["wide"]
    engine = ContinuousBatchingEngine(load(folder, dtype), KVConfig(block_size=32), num_blocks=12,
                                      max_batch_tokens=48, chunk_size=20, max_num_seqs=3)
    reqs = []
    for i, n in enumerate([1, 9, 40, 64, 9, 70, 2]):
        prompt = ru.random_ids(n, config["vocab"], 400 + i)
        reqs.append((engine.add_request(prompt, 9, SamplingParams(temperature=0.0)), prompt))
    engine.run_until_done()
    out = engine.collect_outputs()
    for rid, prompt in reqs:
        assert len(out[rid]) == 9
        assert_greedy(weights, config, prompt, out[rid], dtype)
    assert engine.runner.cache.free_slots() == 3


# ----------------------------------------------------------------------- kernels one by one
def dev(t, dtype=torch.float32):
    return t.to(device="cuda:0", dtype=dtype).contiguous()


@pytest.mark.parametrize("width", [52, 256, 1000])
def test_sum_norm_kernel(width):
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(width)
    x, d = torch.randn(7, width, generator=g), torch.randn(7, width, generator=g)
    w = 1 + 0.1 * torch.randn(width, generator=g)
    want = plain.rms_norm(1.7 * x.double() + d.double(), w.double(), 1e-5)
    full, rounded = norm32.sum_norm(dev(x), dev(w), 1e-5, delta=dev(d, torch.bfloat16).float(), alpha=1.7,
                                    out_dtype=torch.bfloat16)
    want16 = plain.rms_norm(1.7 * x.double() + d.bfloat16().double(), w.double(), 1e-5)
    assert (full.cpu().double() - want16).abs().max() < 1e-5
    assert (rounded.float().cpu().double() - want16).abs().max() < 0.02
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda:0")
    _, picked = norm32.sum_norm(dev(x), dev(w), 1e-5, rows=rows, out_dtype=torch.float32, want32=False)
    assert (picked.cpu().double() - plain.rms_norm(x.double(), w.double(), 1e-5)[[5, 0, 5]]).abs().max() < 1e-5
    del want


def test_head_norm_gate_and_xielu_kernels():
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(4)
    T, H, dv = 5, 3, 20
    o, gate, gain = torch.randn(T, H * dv, generator=g) * 3, torch.randn(T, H * dv, generator=g), torch.rand(dv, generator=g)
    y = norm32.head_norm_gate(dev(o), H, 1e-6, torch.float32, gain=dev(gain), gate=dev(gate))
    want = plain.rms_norm(o.double().view(T, H, dv), gain.double(), 1e-6).reshape(T, -1) * torch.nn.functional.silu(gate.double())
    assert (y.cpu().double() - want).abs().max() < 1e-5
    y = norm32.head_norm_gate(dev(o), H, 1e-6, torch.float32)
    assert (y.cpu().double() - plain.rms_norm(o.double().view(T, H, dv), None, 1e-6).reshape(T, -1)).abs().max() < 1e-5
    z = torch.cat([torch.randn(4, 33, generator=g) * 3, torch.zeros(1, 33)])
    pq = torch.tensor([0.4, -0.7])
    got = norm32.xielu(dev(z), dev(pq), torch.float32)
    assert (got.cpu().double() - plain.xielu(z.double(), pq[0].double(), pq[1].double())).abs().max() < 1e-5


@pytest.mark.parametrize("H,d,dv", [(1, 10, 7), (2, 64, 48), (2, 160, 40), (3, 32, 130)])
@pytest.mark.parametrize("mode", ["decay", "gate"])
def test_recurrence_kernel_carries_its_state_over_cuts(H, d, dv, mode):
    """Two requests of unequal length, run whole, and again cut at arbitrary places with the
    other request's slot in between: outputs and final states agree with the plain recurrence."""
    from dispec_b200.ops import recurrence as R
    g = torch.Generator().manual_seed(H * 100 + d)
    lens, slots = [37, 5], [2, 0]
    cols = 2 * H * d + H * dv
    proj = [torch.randn(n, cols, generator=g) for n in lens]
    decay = torch.tensor([0.9, 1.0, 0.99][:H])
    bias, lower = torch.randn(H * d, generator=g), torch.rand(H * d, generator=g)
    rot = (d // 2) * 2 - 2 if d > 4 else 0
    inv_freq = (100.0 ** (-torch.arange(0, rot, 2).double() / max(rot, 1))).float()

    def plain_run(p):
        n = p.shape[0]
        q, k, v = p[:, :H * d].double().view(n, H, d), p[:, H * d:2 * H * d].double().view(n, H, d), p[:, 2 * H * d:].double().view(n, H, dv)
        S, out = torch.zeros(H, d, dv, dtype=torch.float64), []
        for t in range(n):
            if mode == "decay":
                pos = torch.tensor([t])
                qt = plain.rotate_halves(q[t:t + 1], pos, 100.0, rot)[0] if rot else q[t]
                kt = (plain.rotate_halves(k[t:t + 1], pos, 100.0, rot)[0] if rot else k[t]) * d ** -0.5
                S = decay.double()[:, None, None] * S + kt[:, :, None] * v[t][:, None, :]
            else:
                qt = torch.nn.functional.silu(q[t])
                f = (lower.double() + (1 - lower.double()) * torch.sigmoid(k[t].reshape(-1) + bias.double())).view(H, d)
                S = f[:, :, None] * S + (1 - f)[:, :, None] * v[t][:, None, :]
            out.append(torch.einsum("hdv,hd->hv", S, qt).reshape(-1))
        return torch.stack(out), S

    want = [plain_run(p) for p in proj]
    kw = (dict(decay=dev(decay), inv_freq=dev(inv_freq) if rot else None, rot=rot, key_scale=d ** -0.5) if mode == "decay"
          else dict(gate_bias=dev(bias), lower=dev(lower)))
    code = R.FIXED_DECAY if mode == "decay" else R.FORGET_GATE
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda:0")
    for cuts in ([[37], [5]], [[2, 16, 1, 18], [3, 2]]):
        state = torch.full((4, H, d, dv), float("nan"), device="cuda:0")
        state[slots] = 0.0
        got = [[], []]
        done = [0, 0]
        for step in range(max(len(c) for c in cuts)):
            rows, starts, sl, pos, who = [], [0], [], [], []
            for s in (1, 0):  # the shorter request first
                if step < len(cuts[s]):
                    n = cuts[s][step]
                    rows.append(proj[s][done[s]:done[s] + n])
                    pos += list(range(done[s], done[s] + n))
                    starts.append(starts[-1] + n)
                    sl.append(slots[s])
                    who.append((s, n))
                    done[s] += n
            o = R.linear_recurrence(dev(torch.cat(rows)), 0, H * d, 2 * H * d, code, H, d, dv, state, i32(sl),
                                    i32(starts), i32(pos), **kw)
            at = 0
            for s, n in who:
                got[s].append(o[at:at + n].cpu())
                at += n
        for s in (0, 1):
            o = torch.cat(got[s]).double()
            tol = 1e-4 * max(1.0, want[s][0].abs().max().item())
            assert (o - want[s][0]).abs().max() < tol, (cuts, s)
            assert (state[slots[s]].cpu().double() - want[s][1]).abs().max() < tol
        assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all()  # other slots untouched
    # a sequence whose first position is negative (a padding row) leaves its slot alone
    before = state.clone()
    R.linear_recurrence(dev(proj[1][:1]), 0, H * d, 2 * H * d, code, H, d, dv, state, i32([0]), i32([0, 1]), i32([-1]), **kw)
    assert torch.equal(torch.nan_to_num(state), torch.nan_to_num(before))


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,r,page", [(3, 20, 6, 8), (10, 192, 16, 16), (2, 520, 64, 64)])
def test_latent_attention_kernel_sees_exactly_the_causal_keys(H, R, r, page, pool_dtype):
    """One key's score stands out by far: the first token, keys on both sides of page borders, the
    query's own position, and the position after it (stored already, as in a portion of a prompt:
    it must stay invisible).  Pages are scattered over the pool; the rest of the pool is NaN."""
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(R)
    n = 5 * page + 3  # stored tokens
    n_pages = 9
    table = torch.tensor([[7, 2, 5, 0, 8, 3]], dtype=torch.int32)
    lat = torch.randn(n, R, generator=g).to(pool_dtype).float()
    rk = torch.randn(n, r, generator=g).to(pool_dtype).float()
    c_pool = torch.full((n_pages, 1, page, R), float("nan"))
    r_pool = torch.full((n_pages, 1, page, r), float("nan"))
    for j in range(n):
        c_pool[table[0, j // page], 0, j % page] = lat[j]
        r_pool[table[0, j // page], 0, j % page] = rk[j]
    qpos = [n - 2, n - 2, n - 2, n - 2, n - 2, n - 2, page, 0]
    star = [0, page - 1, page, 3 * page + 1, n - 2, n - 1, page, 0]  # the key each query is aimed at
    T = len(qpos)
    rot = r - 2 if r > 2 else r
    inv_freq = (50.0 ** (-torch.arange(0, rot, 2).double() / rot)).float()
    qa = torch.randn(T, H, R, generator=g) * 0.05
    q_rot = torch.randn(T, H, r, generator=g) * 0.05
    for t in range(T):
        qa[t] += 6.0 * lat[star[t]] / lat[star[t]].norm() ** 2 * math.sqrt(R)
    qraw = torch.zeros(T, H * (5 + r))
    for a in range(H):
        qraw[:, a * (5 + r) + 5:(a + 1) * (5 + r)] = q_rot[:, a]
    scale = 0.37
    out = LO.latent_attention(dev(qa.reshape(T, -1)), dev(qraw), 5 + r, 5, dev(inv_freq), rot, dev(c_pool, pool_dtype),
                              dev(r_pool, pool_dtype), table.to("cuda:0").expand(T, -1).contiguous(),
                              torch.tensor(qpos, dtype=torch.int32, device="cuda:0"),
                              torch.arange(T, dtype=torch.int32, device="cuda:0"), H, scale, torch.float32)
    out = out.cpu().double().view(T, H, R)
    for t in range(T):
        p = qpos[t]
        qr = plain.rotate_interleaved(q_rot[t].double()[None], torch.tensor([p]), 50.0, rot)[0]
        s = (qa[t].double() @ lat[:p + 1].double().T + qr @ rk[:p + 1].double().T) * scale
        w = torch.softmax(s, dim=-1)
        want = w @ lat[:p + 1].double()
        assert (out[t] - want).abs().max() < 2e-4, (t, star[t])
        if star[t] <= p:
            assert w[:, star[t]].min() > 0.5  # the aimed-at key does carry the result
        else:
            assert w.max() < 0.9  # the stored but invisible key: nothing stands out among the visible


def test_latent_store_kernel_norms_rotates_and_places():
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(2)
    R, r, page, Q = 20, 8, 4, 3
    down = torch.randn(6, Q + R + r, generator=g)
    gain = torch.rand(R, generator=g) + 0.5
    pos = torch.tensor([3, 4, 5, 0, -1, 9], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    table = torch.tensor([[2, 0, -1], [1, 3, 4]], dtype=torch.int32)
    rot = 6
    inv_freq = (20.0 ** (-torch.arange(0, rot, 2).double() / rot)).float()
    c_pool = torch.full((5, 1, page, R), float("nan"), device="cuda:0")
    r_pool = torch.full((5, 1, page, r), float("nan"), device="cuda:0")
    LO.latent_store(dev(down), Q, Q + R, dev(gain), 1e-6, dev(inv_freq), rot, pos.cuda(), seq.cuda(), table.cuda(),
                    c_pool, r_pool)
    written = 0
    for t in range(6):
        if pos[t] < 0:
            continue
        pg, off = int(table[seq[t], pos[t] // page]), int(pos[t] % page)
        c = plain.rms_norm(down[t, Q:Q + R].double(), gain.double(), 1e-6)
        k = plain.rotate_interleaved(down[t, Q + R:].double()[None, None], pos[t:t + 1], 20.0, rot)[0, 0]
        assert (c_pool[pg, 0, off].cpu().double() - c).abs().max() < 1e-5
        assert (r_pool[pg, 0, off].cpu().double() - k).abs().max() < 1e-5
        written += 1
    assert int(torch.isfinite(c_pool[:, 0, :, 0]).sum()) == written  # nothing else was touched


@pytest.mark.parametrize("H,R,r,page", [(10, 192, 16, 16), (12, 512, 64, 16), (70, 64, 32, 8), (3, 128, 0, 32),
                                        (5, 256, 48, 16), (2, 384, 16, 64), (4, 128, 32, 16)])
def test_latent_attention_on_tensor_cores_matches_the_plain_softmax(H, R, r, page):
    """The tensor-core kernel over a step of two single tokens (keys cut into ranges and merged)
    and a portion of a prompt whose tiles end in the middle of a key tile; every query is aimed at
    one key: the first, both sides of a page border, its own position, or the next one (stored,
    invisible).  Scattered pages, NaN everywhere else."""
    from types import SimpleNamespace
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(H + R)
    lens = [3 * page + 5, 200, 9 * page + 7]  # stored tokens per request; the third brings a portion
    portion = 45
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    tables, lat, rk = [], [], []
    width = max(-(-n // page) for n in lens)
    c_pool = torch.full((n_pages, 1, page, R), float("nan"))
    r_pool = torch.full((n_pages, 1, page, max(r, 1)), float("nan"))[..., :r]
    for n in lens:
        need = -(-n // page)
        tables.append([perm.pop() for _ in range(need)] + [-1] * (width - need))
        lat.append(torch.randn(n, R, generator=g).bfloat16().float())
        rk.append(torch.randn(n, r, generator=g).bfloat16().float())
        for j in range(n):
            c_pool[tables[-1][j // page], 0, j % page] = lat[-1][j]
            r_pool[tables[-1][j // page], 0, j % page] = rk[-1][j]
    q_lens = [1, 1, portion]
    seq_of, pos = [], []
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        seq_of += [s] * ql
        pos += list(range(n - ql, n))
    T = len(pos)
    aims = [0, page - 1, page, None, "self", "next"]
    star = []
    for t in range(T):
        a = aims[t % len(aims)]
        n = lens[seq_of[t]]
        star.append(a if isinstance(a, int) else pos[t] if a == "self" else min(pos[t] + 1, n - 1) if a == "next" else pos[t] // 2)
    rot = r
    inv_freq = (50.0 ** (-torch.arange(0, max(rot, 2), 2).double() / max(rot, 1))).float()
    qa = torch.randn(T, H, R, generator=g) * 0.05
    q_rot = torch.randn(T, H, r, generator=g) * 0.05
    for t in range(T):
        c = lat[seq_of[t]][star[t]]
        qa[t] += 8.0 * c / c.norm() ** 2 * math.sqrt(R)
    qraw = torch.zeros(T, H * (8 + r))
    for a in range(H):
        qraw[:, a * (8 + r) + 8:(a + 1) * (8 + r)] = q_rot[:, a]
    qraw = qraw.bfloat16()
    tpt = LO.mma_tokens_per_tile(H)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda:0")
    tiles = [(s, a) for s, ql in enumerate(q_lens) for a in range(0, ql, tpt)]
    ctx = SimpleNamespace(attention_tiles={tpt: (i32([s for s, _ in tiles]), i32([a for _, a in tiles]), len(tiles))},
                          q_start=i32([0, 1, 2, 2 + portion]), ctx_len=i32(lens), num_decode_seqs=2, max_ctx_len=max(lens))
    assert LO.mma_supported(R, r, torch.bfloat16)
    scale = 0.21
    out = LO.latent_attention_tiles(ctx, dev(qa.reshape(T, -1)), dev(qraw, torch.bfloat16), 8 + r, 8, dev(inv_freq), rot,
                                    dev(c_pool, torch.bfloat16), dev(r_pool, torch.bfloat16), i32(tables), H, scale)
    out = out.float().cpu().double().view(T, H, R)
    assert torch.isfinite(out).all()
    for t in range(T):
        s_, p = seq_of[t], pos[t]
        qr = q_rot[t].bfloat16().double()
        if rot:
            qr = plain.rotate_interleaved(qr[None], torch.tensor([p]), 50.0, rot)[0]
        sc = (qa[t].double() @ lat[s_][:p + 1].double().T + qr @ rk[s_][:p + 1].double().T) * scale
        w = torch.softmax(sc, dim=-1)
        want = w @ lat[s_][:p + 1].double()
        assert (out[t] - want).abs().max() < 0.05 * max(1.0, want.abs().max().item()), (t, star[t], p)


@pytest.mark.parametrize("M,H,N,K,out_dtype", [(5, 3, 40, 32, torch.float32), (200, 12, 128, 512, torch.bfloat16),
                                               (130, 2, 192, 64, torch.float32)])
def test_head_products_kernel(M, H, N, K, out_dtype):
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(M)
    pad = 8  # columns between the heads' blocks of x that the product must not read
    x = torch.randn(M, H * (K + pad), generator=g).bfloat16()
    w = (torch.randn(H, N, K, generator=g) / K ** 0.5).bfloat16()
    out = torch.full((M, H * N + 3), float("nan"), dtype=out_dtype, device="cuda:0")
    xd, wd = x.cuda(), w.cuda()
    assert LO.head_products_supported(xd, K + pad, wd)
    LO.head_products(xd, K + pad, wd, out, N)
    for a in range(H):
        want = x[:, a * (K + pad):a * (K + pad) + K].double() @ w[a].double().T
        got = out[:, a * N:(a + 1) * N].double().cpu()
        tol = 1e-4 if out_dtype == torch.float32 else 0.02
        assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item()), a
    assert torch.isnan(out[:, H * N:]).all()
