"""The Tutizen decoder in the engine against the plain float64 implementation (``plain_tutizen``): each mechanism alone
and in a model of its own, whole prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests on pages that are used again, far keys that only the heads with small slopes still see, keys at page
borders, the first tokens, long decoding, sizes unlike one another (one key head, values wider or narrower than keys,
borrowed pages, no feed-forward, one choice, no groups, no shared expert, sizes that are multiples of 2 only), the
tensor-core attention kernels against the exact one, and greedy generation through the engine's scheduler."""

import copy

import pytest
import torch

import plain_tutizen as plain
import trace_modes as modes
import tutizen_cases as cases
from helpers import compare_logits, seeded_tokens, write_model_dir

pytestmark = pytest.mark.gpu
STORED = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= tol * scale, f"max abs error {err:.3e} against scale {scale:.3e}"


def compare_rows(got, want, dtype):
    """float32: the helpers' bound (cosine and largest difference). bfloat16: what the rounding of activations leaves of
    a row, a few per cent of its spread for these small random models; a wrong key, slope or expert changes a row
    outright, and the float32 runs of the same cuttings hold the tight bound."""
    if dtype == "float32":
        return compare_logits(got, want, dtype)
    a, b = got.double().reshape(-1), want.double().reshape(-1)
    if not torch.isfinite(a).all():
        return False, "non-finite logits"
    cos = float(torch.nn.functional.cosine_similarity(a, b, dim=0))
    rel = float((a - b).norm() / (b - b.mean()).norm())
    return cos >= 0.998 and rel <= 0.06, f"cosine {cos:.6f}, error {rel:.3f} of the row's spread"


def rounded(state, dtype):
    return {k: v.to(STORED[dtype]) for k, v in state.items()}


def replay(folder, dtype, steps, want, page, slots, label, poison=True, min_ok=1.0):
    """Runs the steps through a fresh session and compares every wanted row; pages start as NaN."""
    from stride_b200.engine.trace import TraceSession
    session = TraceSession(folder, dtype, max_tokens=modes.peak_tokens(steps), block_size=page, max_requests=slots)
    if poison:
        for t in session.device_cache.pages:
            t.fill_(float("nan"))
    rows = modes.expected_rows(steps)
    bad, total, first = 0, 0, None
    for s in steps:
        out = session.run_step(s)
        for r, (rid, pos) in enumerate(rows[s["step"]]):
            ok, msg = compare_rows(out[r:r + 1], want[rid][pos:pos + 1], dtype)
            total += 1
            if not ok:
                bad += 1
                first = first or f"{label}: step {s['step']}, request {rid!r}, position {pos}: {msg}"
    assert total and bad <= (1.0 - min_ok) * total, f"{bad} of {total} rows differ; first: {first}"
    stats = session.cache.stats()
    assert stats["live"] == 0 and session.cache.free_slots == session.cache.slot_capacity
    return session


def model_case(tmp_models, name, cfg, dtype, seed, lengths):
    state = cases.seeded_state(cfg, seed)
    folder = write_model_dir(str(tmp_models / f"tutizen_{name}_{dtype}_{seed}"), cfg, state, STORED[dtype])
    state = {k: v.double() for k, v in rounded(state, dtype).items()}
    requests = {f"r{i}": seeded_tokens(n, cfg["vocab"], 50 * seed + i) for i, n in enumerate(lengths)}
    want = {rid: plain.forward(cfg, state, toks) for rid, toks in requests.items()}
    return folder, requests, want


# ------------------------------------------------------------------------------------------- small kernels
@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1e-2)])
@pytest.mark.parametrize("width,with_bias", [(54, True), (64, False), (344, True), (2048, True), (1032, False), (4104, True)])
def test_norm_on_a_sublayers_output(gpu, dtype, tol, width, with_bias):
    """x + m g unit_rms(y + b) through the part, with the copy that the next sublayer reads."""
    from stride_b200.config import NormSpec
    from stride_b200.parts import ResidualStream, Runtime, build_part
    rt = Runtime("cuda", STORED[dtype], 16, 4)
    g = torch.Generator().manual_seed(width)
    norm = build_part("norm", NormSpec("rmsnorm", width, 1e-3, "n", (("tensor", "n"), ("shape", "scalar"))), rt)
    assert norm.declare()["n"].shape == ()
    gain = torch.tensor(1.3)
    norm.bind({"n": gain.cuda()})
    assert norm.named_tensors()["n"].shape == ()
    x, y = torch.randn(6, width, generator=g), (torch.randn(6, width, generator=g) * 5).to(STORED[dtype])
    bias = torch.randn(width, generator=g) if with_bias else None
    stream = ResidualStream(rt, 6, width)
    stream.residual.copy_(x)
    first = stream.values()
    close(first, x.double(), tol)
    stream.add_normed(y.cuda(), norm, 0.7, bias.cuda() if with_bias else None)
    want = x.double() + 0.7 * plain.scalar_norm(y.double() + (bias.double() if with_bias else 0.0), gain.double(), 1e-3)
    close(stream.materialize(), want, 3e-6)
    stream.add_normed(y.cuda(), norm, 0.7, None)
    close(stream.values(), want + 0.7 * plain.scalar_norm(y.double(), gain.double(), 1e-3), tol)
    # as a norm before the head: the one number is spread over the width
    close(stream.normed(norm, rows=torch.tensor([4, 1], dtype=torch.int32, device="cuda")),
          plain.scalar_norm(stream.materialize().double().cpu()[[4, 1]], gain.double(), 1e-3), tol)


@pytest.mark.parametrize("width", [10, 33, 128])
def test_position_vectors(gpu, width):
    from stride_b200.csrc import ops
    positions = [0, 1, 2, 63, 64, 1000, 4097, 30011]
    x = torch.zeros(len(positions) + 1, width, device="cuda")
    copy_ = torch.zeros(len(positions) + 1, width, dtype=torch.bfloat16, device="cuda")
    freq = 10000.0 ** (-2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    ops.add_sinusoid(x, copy_, dev(positions + [7]), dev([0] * len(positions) + [-1]), freq.cuda())
    want = plain.position_vectors(positions, width)
    assert (x[:-1].double().cpu() - want).abs().max() < 1e-7        # float64 angles: exact to float32 rounding at any position
    assert float(x[-1].abs().max()) == 0.0                          # a padded row stays as it is
    close(copy_[:-1], want, 1e-2)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1e-2)])
@pytest.mark.parametrize("nq,nkv,hd,vd,extra", [(3, 1, 32, 32, 8), (4, 4, 16, 24, 0), (2, 2, 48, 16, 8), (3, 3, 20, 18, 3), (2, 1, 128, 256, 0)])
def test_head_norms_and_the_cache_write(gpu, dtype, tol, nq, nkv, hd, vd, extra):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(hd + vd)
    tokens, page, pages = 11, 4, 9
    cols = (nq + nkv) * hd + nkv * vd
    raw = (torch.randn(tokens, cols + extra, generator=g) * 3).to(STORED[dtype])
    bias = torch.randn(cols, generator=g)
    slots = torch.randperm(page * pages, generator=g)[:tokens].to(torch.int32)
    k_pages = torch.full((pages, nkv, page, hd), 7.0, dtype=STORED[dtype], device="cuda")
    v_pages = torch.full((pages, nkv, page, vd), 7.0, dtype=STORED[dtype], device="cuda")
    qkv = raw.cuda()
    ops.qkv_unit_norm(qkv, bias.cuda(), slots.cuda(), k_pages, v_pages, nq, nkv, hd, vd, page, 1e-4)
    y = raw[:, :cols].double() + bias.double()
    q = plain.unit_rms(y[:, :nq * hd].view(tokens, nq, hd), 1e-4)
    k = plain.unit_rms(y[:, nq * hd:(nq + nkv) * hd].view(tokens, nkv, hd), 1e-4)
    v = plain.unit_rms(y[:, (nq + nkv) * hd:].view(tokens, nkv, vd), 1e-4)
    close(qkv[:, :nq * hd], q.reshape(tokens, -1), tol)
    if extra:
        assert torch.equal(qkv[:, cols:].cpu(), raw[:, cols:])             # what lies behind the heads is left alone
    for t in range(tokens):
        s = int(slots[t])
        close(k_pages[s // page, :, s % page], k[t], tol)
        close(v_pages[s // page, :, s % page], v[t], tol)
    used = torch.zeros(pages * page, dtype=torch.bool)
    used[slots.long()] = True
    untouched = k_pages.permute(0, 2, 1, 3).reshape(pages * page, -1)[~used]
    assert bool((untouched == 7.0).all())
    # queries alone (a layer that borrows its pages), and with the norms switched off: only the bias is added
    alone = raw[:, :nq * hd + extra].contiguous().cuda()
    ops.qkv_unit_norm(alone, bias[:nq * hd].contiguous().cuda(), None, None, None, nq, 0, hd, vd, page, 1e-4)
    close(alone[:, :nq * hd], q.reshape(tokens, -1), tol)
    plain_sum = raw.cuda()
    ops.qkv_unit_norm(plain_sum, bias.cuda(), None, None, None, nq, nkv, hd, vd, page, 1e-4, False, False)
    close(plain_sum[:, :cols], y, tol)


def test_one_gate_per_head(gpu):
    """Head widths that are whole 16-byte packs (the vector kernel) and one that is not; the gates stand in a column block of a wider buffer."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 1e-2)):
        for tokens, heads, width in ((5, 3, 10), (7, 3, 16), (300, 5, 64), (2, 1, 8)):
            x, wide = torch.randn(tokens, heads * width, generator=g).to(dtype), (torch.randn(tokens, 17, generator=g) * 3).to(dtype)
            a, w = x.cuda(), wide.cuda()
            ops.head_gate(a, w[:, 9:], 17, heads, width)
            want = x.double().view(tokens, heads, width) * torch.sigmoid(wide.double()[:, 9:9 + heads])[:, :, None]
            close(a, want.reshape(tokens, heads * width), tol)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1e-2)])
@pytest.mark.parametrize("tokens,inter,block", [(7, 48, 48), (5, 128, 64), (3, 30, 6)])
def test_clamped_gate_times_up(gpu, dtype, tol, tokens, inter, block):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(inter)
    gate, up = (torch.randn(tokens, inter, generator=g).to(STORED[dtype]) * 2 for _ in range(2))         # many values beyond the limit
    stacked = torch.stack([gate.view(tokens, inter // block, block), up.view(tokens, inter // block, block)], dim=2).reshape(tokens, 2 * inter)
    out = torch.empty(tokens, inter, dtype=STORED[dtype], device="cuda")
    ops.gated_act(stacked.contiguous().cuda(), out, block, "swish_clamped", 1.25, 1.702)
    gg, uu = gate.double().clamp(max=1.25), up.double().clamp(-1.25, 1.25)
    close(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), tol)


@pytest.mark.parametrize("tokens,inter,k,limit", [(8, 9600, 512, 7.0), (3, 960, 192, 0.8), (1, 14336, 448, 1.25)])
def test_clamped_activation_in_the_epilogue_of_the_gate_and_up_product(gpu, tokens, inter, k, limit):
    """The product for a few tokens that applies the clamped activation itself, against the product followed by the kernel above."""
    from stride_b200.csrc import ops
    from stride_b200.parts.swiglu import interleave_gate_up
    g = torch.Generator().manual_seed(inter)
    x = torch.randn(tokens, k, generator=g).bfloat16().cuda()
    gate, up = ((torch.randn(inter, k, generator=g) * (2.0 / k ** 0.5)).bfloat16() for _ in range(2))      # products of spread 2: many beyond a small limit
    w = interleave_gate_up(gate, up, ops.GATED_BLOCK).cuda()
    out = torch.full((tokens, inter), 7.0, dtype=torch.bfloat16, device="cuda")
    if not ops.linear_gated_tc(x, w, out, None, "swish_clamped", limit, 1.702):
        pytest.skip("the tcgen05 product does not take these sizes")
    both = torch.empty(tokens, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.linear(x, w, both)
    unfused = torch.empty_like(out)
    ops.gated_act(both, unfused, ops.GATED_BLOCK, "swish_clamped", limit, 1.702)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    close(out, unfused, 1e-2)
    gx = (x.double().cpu() @ gate.double().T).bfloat16().double().clamp(max=limit)
    ux = (x.double().cpu() @ up.double().T).bfloat16().double().clamp(-limit, limit)
    close(out, gx * torch.sigmoid(1.702 * gx) * (ux + 1.0), 1e-2)


@pytest.mark.parametrize("n,k,act,out_dtype", [(96, 72, 2, torch.bfloat16), (256, 64, 2, torch.bfloat16), (130, 200, 0, torch.float32),
                                               (384, 136, 1, torch.bfloat16), (64, 1024, 0, torch.float32), (20, 8, 2, torch.float32)])
def test_expert_products_on_the_tcgen05_tiles(gpu, n, k, act, out_dtype):
    """Rows lying expert by expert, with experts of no row, one row, exactly one tile and several ragged tiles: the
    tcgen05 grouped product against float64, and against the mma.sync tiles; rows it must not touch keep their value."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(n * k + act)
    counts = [0, 1, 128, 300, 0, 129, 77, 0]
    offsets = torch.tensor([0] + torch.tensor(counts).cumsum(0).tolist(), dtype=torch.int32)
    rows, spare = int(offsets[-1]), 40
    a = torch.randn(rows + spare, k, generator=g).bfloat16()
    w = (torch.randn(len(counts), n, k, generator=g) * (1.5 / k ** 0.5)).bfloat16()
    width = n // 2 if act == 2 else n
    out = torch.full((rows + spare, width), 3.0, dtype=out_dtype, device="cuda")
    if not ops.grouped_gemm_tc(a.cuda(), w.cuda(), offsets.cuda(), out, rows + spare, act, 0.9, 1.702):
        pytest.skip("the tcgen05 grouped product does not take these sizes")
    tiles = torch.full_like(out, 3.0)
    ops.grouped_gemm(a.cuda(), None, w.cuda(), offsets.cuda(), tiles, rows + spare, act, 0.9, 1.702)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    want = torch.full((rows + spare, width), 3.0, dtype=torch.float64)
    for e, c in enumerate(counts):
        lo = int(offsets[e])
        z = a[lo:lo + c].double() @ w[e].double().T
        if act == 1:
            z = z.clamp(min=0) ** 2
        elif act == 2:
            gg, uu = z[:, 0::2].clamp(max=0.9), z[:, 1::2].clamp(-0.9, 0.9)
            z = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)
        want[lo:lo + c] = z
    tol = 1e-2 if out_dtype == torch.bfloat16 else 2e-5
    close(out, want, tol)
    close(out, tiles, tol)
    assert torch.equal(out[rows:].cpu().double(), want[rows:]), "rows past the last expert's were written"


def test_rows_laid_out_expert_by_expert(gpu):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    x = torch.randn(50, 72, generator=g).bfloat16()
    perm = torch.randint(0, 50, (90,), generator=g, dtype=torch.int32)
    offsets = torch.tensor([0, 30, 30, 81], dtype=torch.int32)          # 81 rows filled of room for 90
    xs = torch.full((90, 72), 5.0, dtype=torch.bfloat16, device="cuda")
    assert ops.gather_rows(x.cuda(), perm.cuda(), offsets.cuda(), 3, xs, 90)
    torch.cuda.synchronize()
    assert torch.equal(xs[:81].cpu(), x[perm[:81].long()]) and bool((xs[81:] == 5.0).all())


@pytest.mark.parametrize("experts,top,groups,keep", [(10, 2, 5, 3), (8, 2, 4, 2), (6, 3, 1, 1), (4, 1, 2, 2), (9, 2, 3, 1), (64, 6, 8, 3), (256, 8, 8, 4),
                                                     (5, 5, 5, 5), (6, 2, 6, 2)])
def test_router_with_sigmoid_scores_and_groups(gpu, experts, top, groups, keep):
    """Against the plain rule, with corrections that reorder the scores and make choice scores negative; the logits ride in
    a wider buffer, as the part lays them out."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(experts * top)
    tokens, width = 67, 24
    x = torch.randn(tokens, width, generator=g)
    w = {"p.router": torch.randn(experts, width, generator=g) * 0.5, "p.correction": torch.randn(experts, generator=g) * 0.8 - 0.7}
    logits = torch.zeros(tokens, experts + 3)
    logits[:, :experts] = (x.double() @ w["p.router"].double().T).float()
    router = {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}
    # the plain rule on the same float32 logits (sigmoid is monotone: x with an identity router gives them back)
    want_ids, want_w = plain.route(logits[:, :experts].double(), {"p.router": torch.eye(experts, dtype=torch.float64),
                                                                  "p.correction": w["p.correction"].double()}, "p.", router)
    ids = torch.full((tokens + 1, top), -5, dtype=torch.int32, device="cuda")
    weights = torch.zeros(tokens + 1, top, device="cuda")
    seq = torch.zeros(tokens + 1, dtype=torch.int32, device="cuda")
    seq[-1] = -1
    ops.moe_select_sigmoid(torch.cat([logits, logits[:1]]).cuda(), w["p.correction"].cuda(), seq, ids, weights, experts, groups, keep, 2.5)
    assert ids[:tokens].cpu().tolist() == want_ids
    close(weights[:tokens], torch.tensor([[float(a) for a in row] for row in want_w], dtype=torch.float64), 1e-5)
    assert ids[-1].cpu().tolist() == [-1] * top and float(weights[-1].abs().max()) == 0.0


def test_router_keeps_negative_choice_scores_out_of_dropped_groups(gpu):
    """Every choice score is negative and the largest ones sit in a group that is dropped: counting dropped experts as 0
    would choose them."""
    from stride_b200.csrc import ops
    logits = torch.tensor([[-3.0, -3.0, 2.0, -9.0, 0.5, 0.4, -1.0, -1.2]])
    correction = torch.full((8,), -2.0)
    # choice scores: group 0 about (-1.95, -1.95), group 1 (-1.12, -2.0), group 2 (-1.38, -1.40), group 3 (-1.73, -1.77)
    router = {"experts": 8, "top": 2, "scale": 1.0, "groups": {"count": 4, "keep": 1}}
    want_ids, want_w = plain.route(logits.double(), {"p.router": torch.eye(8, dtype=torch.float64), "p.correction": correction.double()}, "p.", router)
    assert want_ids == [[4, 5]]
    ids, weights = torch.zeros(1, 2, dtype=torch.int32, device="cuda"), torch.zeros(1, 2, device="cuda")
    ops.moe_select_sigmoid(logits.cuda(), correction.cuda(), None, ids, weights, 8, 4, 1, 1.0)
    assert ids.cpu().tolist() == want_ids
    close(weights, torch.tensor([[float(a) for a in row] for row in want_w], dtype=torch.float64), 1e-6)


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("width,ff,experts,top,tokens", [(96, 24, 8, 2, 37), (100, 14, 9, 2, 37), (128, 64, 4, 1, 37), (136, 72, 6, 3, 400),
                                                         (64, 128, 5, 2, 700)])
def test_gated_experts_and_the_gated_shared_expert(gpu, tmp_models, dtype, tol, width, ff, experts, top, tokens):
    """The routed feed-forward as a part, against the plain mixture, for inputs that drive many units into the clamp; the
    steps of many rows run the experts on the tcgen05 tiles in bfloat16."""
    from stride_b200.config import FeedForwardSpec
    from stride_b200.parts import Runtime, build_part
    cfg = cases.config(width, 50, [(cases.attn(1, 1, 8), cases.moe(experts, top, ff, 0.9, groups=None, scale=1.5, shared=(ff + 6, 0.6)))])
    state = {k: v.to(STORED[dtype]) for k, v in cases.seeded_state(cfg, 5).items() if k.startswith("l0.mlp.")}
    rt = Runtime("cuda", STORED[dtype], max(64, tokens), 4)
    part = build_part("feed_forward", FeedForwardSpec("routed_experts", width, ff, "swish_clamped", "l0.mlp.", params=(
        ("experts", experts), ("top", top), ("router", "sigmoid_groups"), ("route_scale", 1.5), ("limit", 0.9), ("alpha", 1.702),
        ("shared", ff + 6), ("shared_limit", 0.6), ("shared_gate", True))), rt)
    assert set(part.declare()) == set(state)
    part.bind({k: (v.float() if v.dim() == 1 else v).cuda() for k, v in state.items()})
    for name, t in part.named_tensors().items():
        assert torch.equal(t.cpu().to(state[name].dtype), state[name]), name
    g = torch.Generator().manual_seed(width)
    x = (torch.randn(tokens, width, generator=g) * 1.5).to(STORED[dtype])

    class Ctx:
        seq_of_token = torch.zeros(max(64, tokens), dtype=torch.int32, device="cuda")
    out = part.forward(x.cuda(), Ctx)
    want = plain.moe_ff(x.double(), {k: v.double() for k, v in state.items()}, "l0.mlp.", cfg["layers"][0]["mlp"])
    close(out, want, tol)


def paged_case(g, lens, page, nkv, hd, vd, dtype=torch.bfloat16):
    """Requests of (cached, new) tokens on shuffled pages: index arrays and random keys and values."""
    total_pages = sum(-(-(c + n) // page) for c, n in lens) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    width = max(-(-(c + n) // page) for c, n in lens)
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    q_start, q_len, ctx_len, seq_of, positions, at = [], [], [], [], [], 0
    for s, (c, n) in enumerate(lens):
        pages = [perm.pop() for _ in range(-(-(c + n) // page))]
        table[s, :len(pages)] = torch.tensor(pages)
        q_start.append(at), q_len.append(n), ctx_len.append(c + n)
        seq_of += [s] * n
        positions += list(range(c, c + n))
        at += n
    k = (torch.randn(total_pages, nkv, page, hd, generator=g) * 0.8).to(dtype).cuda()
    v = (torch.randn(total_pages, nkv, page, vd, generator=g) * 0.8).to(dtype).cuda()
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    return k, v, table.cuda(), dev(q_start), dev(q_len), dev(ctx_len), dev(seq_of), dev(positions), at


def slopes_of(nq):
    return torch.tensor(plain.head_slopes(nq), dtype=torch.float32)


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 1e-2)])
@pytest.mark.parametrize("nq,nkv,hd,vd,page", [(3, 1, 32, 32, 8), (4, 4, 16, 24, 4), (2, 2, 48, 16, 16), (6, 3, 10, 6, 8), (2, 1, 64, 200, 16)])
def test_exact_attention_with_slopes_and_a_value_width_of_its_own(gpu, dtype, tol, nq, nkv, hd, vd, page):
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(nq * hd + vd)
    lens = [(0, 70), (40, 9), (257, 1)]
    k, v, table, _qs, _ql, _cl, seq_of, positions, tokens = paged_case(g, lens, page, nkv, hd, vd, STORED[dtype])
    q = (torch.randn(tokens, nq * hd + 5, generator=g) * 0.9).to(STORED[dtype]).cuda()
    slopes, scale = slopes_of(nq), 0.35
    got = torch.zeros(tokens, nq * vd, dtype=STORED[dtype], device="cuda")
    ops.paged_attention(q, nq * hd + 5, got, k, v, table, seq_of, positions, nq, nkv, hd, page, scale, 0, 0.0, None, slopes.cuda(), vd)
    at = 0
    for s, (cached, n) in enumerate(lens):
        pages = table[s].cpu().tolist()
        for t in (at, at + n - 1):
            pos = cached + (t - at)
            rows = lambda cache, head: torch.stack([cache[pages[j // page], head, j % page] for j in range(pos + 1)]).double().cpu()
            for h in range(nq):
                sc = rows(k, h // (nq // nkv)) @ q[t, h * hd:(h + 1) * hd].double().cpu() * scale
                sc = sc - float(slopes[h]) * (pos - torch.arange(pos + 1, dtype=torch.float64))
                close(got[t, h * vd:(h + 1) * vd], torch.softmax(sc, 0) @ rows(v, h // (nq // nkv)), tol)
        at += n


@pytest.mark.parametrize("nq,nkv,hd,page,window,softcap", [(4, 2, 64, 16, 0, 0.0), (6, 2, 128, 16, 0, 0.0), (3, 1, 64, 8, 70, 4.0), (8, 8, 64, 32, 0, 0.0),
                                                           (16, 1, 128, 64, 0, 0.0)])
def test_tensor_core_attention_with_slopes_against_the_exact_kernel(gpu, nq, nkv, hd, page, window, softcap):
    """Portions and single tokens of four requests in one step, through the tcgen05 kernel, the mma.sync kernel and the
    split decode kernel, queries read from a buffer wider than the heads; the exact kernel (held to the formula above) is
    the reference. Sharp scores, so that the penalty decides which keys count."""
    from stride_b200.csrc import ops
    g = torch.Generator().manual_seed(nq * hd)
    lens = [(0, 150), (40, 9), (130, 1), (257, 1)]               # single tokens last, as the step function lays a batch out
    k, v, table, q_start, q_len, ctx_len, seq_of, positions, tokens = paged_case(g, lens, page, nkv, hd, hd)
    stride = nq * hd + 16                                        # sixteen more columns: one gate per head stands there
    q = (torch.randn(tokens, stride, generator=g) * 0.6).bfloat16().cuda()
    slopes, scale = slopes_of(nq).cuda(), 0.2
    want = torch.zeros(tokens, nq * hd, dtype=torch.bfloat16, device="cuda")
    ops.paged_attention(q, stride, want, k, v, table, seq_of, positions, nq, nkv, hd, page, scale, window, softcap, None, slopes)
    without = torch.zeros_like(want)
    ops.paged_attention(q, stride, without, k, v, table, seq_of, positions, nq, nkv, hd, page, scale, window, softcap, None, None)
    assert float((want.float() - without.float()).abs().max()) > 0.1, "the slopes do not show in this case"
    split = 159
    for prefill in (ops.paged_attention_prefill_tc, ops.paged_attention_prefill):
        got = torch.full((tokens, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        done = prefill(q[:split], stride, got[:split], k, v, table, q_start, q_len, ctx_len, 2, nq, nkv, hd, page, scale, window, softcap, None, slopes)
        if done is False:           # the tcgen05 kernel steps aside for pages it does not take
            continue
        scratch = torch.zeros(ops.decode_scratch_floats(2, nq, nkv, hd, 512), device="cuda")
        ops.paged_attention_decode(q[split:], stride, got[split:], k, v, table, seq_of[split:], positions[split:], scratch, nq, nkv, hd, page,
                                   scale, window, 512, softcap, None, slopes)
        torch.cuda.synchronize()
        ops.check_kernel_status()
        close(got, want, 2e-2)
    # the decode kernel with one gate per head, its logits in the query's row
    gated = torch.full((tokens - split, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    scratch = torch.zeros(ops.decode_scratch_floats(2, nq, nkv, hd, 512), device="cuda")
    ops.paged_attention_decode(q[split:], stride, gated, k, v, table, seq_of[split:], positions[split:], scratch, nq, nkv, hd, page,
                               scale, window, 512, softcap, None, slopes, nq * hd)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    gates = torch.sigmoid(q[split:, nq * hd:nq * hd + nq].double())
    close(gated, (want[split:].double().view(-1, nq, hd) * gates[:, :, None]).reshape(-1, nq * hd), 2e-2)


# ------------------------------------------------------------------- each mechanism in a model of nothing else
ONLY_ATTENTION = cases.config(72, 101, [(cases.attn(3, 1, 24, scale=0.4), None), (cases.attn(2, 2, 8, 12, scale=0.7), None),
                                        (cases.attn(3, 1, 24, scale=0.2, kv_from=0), None)], mult=0.9)
ONLY_DENSE = cases.config(56, 89, [(cases.attn(1, 1, 4), cases.dense(70, 0.4))], mult=1.0)
ONLY_MOE = cases.config(56, 89, [(cases.attn(1, 1, 4), cases.moe(10, 2, 10, 0.8, groups=(5, 3), shared=(18, 0.5))),
                                 (cases.attn(1, 1, 4, kv_from=0), cases.moe(5, 1, 6, 3.0))], mult=0.6)


@pytest.mark.parametrize("name,cfg", [("attention", ONLY_ATTENTION), ("dense", ONLY_DENSE), ("moe", ONLY_MOE)])
def test_each_mechanism_in_a_model_of_its_own(gpu, tmp_models, name, cfg):
    folder, requests, want = model_case(tmp_models, name, cfg, "float32", 7, [45, 19, 3])
    replay(folder, "float32", modes.whole(requests), want, 8, 2, name + " whole")
    replay(folder, "float32", modes.changing_portions(requests), want, 8, 2, name + " portions")
    replay(folder, "float32", modes.tail_one_by_one(requests, tail=15), want, 8, 2, name + " decode")


def test_the_stream_after_every_layer(gpu, tmp_models):
    """Layer by layer in float32: the first layer that differs names the mechanism."""
    from stride_b200.engine.trace import TraceSession
    cfg = cases.CASE_A
    state = cases.seeded_state(cfg, 3)
    folder = write_model_dir(str(tmp_models / "tutizen_layers"), cfg, state, torch.float32)
    tokens = seeded_tokens(29, cfg["vocab"], 4)
    want = []
    plain.forward(cfg, {k: v.double() for k, v in state.items()}, tokens, capture=want)
    session = TraceSession(folder, "float32", max_tokens=64, block_size=8, max_requests=1)
    session.model.capture = []
    session.run_step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [0]}], "end": ["a"]})
    assert len(session.model.capture) == len(want)
    for i, (got, expected) in enumerate(zip(session.model.capture, want)):
        err = float((got.double().cpu() - expected).abs().max())
        assert err <= 2e-5 * float(expected.abs().max()), f"the stream differs after layer {i}: {err:.3e}"


# ---------------------------------------------------------------------------- whole models, every cutting
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case,page", [("A", 16), ("B", 8), ("C", 16), ("D", 32)])
def test_every_cutting_gives_the_plain_logits(gpu, tmp_models, case, page, dtype):
    cfg = cases.CASES[case]
    folder, requests, want = model_case(tmp_models, case, cfg, dtype, 11, [90, 33, 1, 52, 9, 2])
    # bfloat16: a router's close call may fall the other way on rounded activations, which changes a row outright
    share = 1.0 if dtype == "float32" else 0.9
    replay(folder, dtype, modes.whole(requests), want, page, 2, "whole", min_ok=share)
    session = replay(folder, dtype, modes.tail_one_by_one(requests, tail=40), want, page, 2, "decode", min_ok=share)
    assert session.runner.graph_replays > 0, "single-token steps did not go through captured graphs"
    replay(folder, dtype, modes.changing_portions(requests), want, page, 2, "portions", min_ok=share)
    # three live requests, six requests in all: pages are used again
    replay(folder, dtype, modes.mixed(requests, live_limit=3, seed=5), want, page, 3, "mixed", min_ok=share)
    replay(folder, dtype, modes.decoding_together(dict(list(requests.items())[:4]), decode_steps=6, prompts_per_step=2), want, page, 4,
           "decoding together", min_ok=share)


def test_float32_logits_do_not_depend_on_the_cutting(gpu, tmp_models):
    """Bitwise: every sum of the 32-bit path has an order that depends on the token's position only."""
    from stride_b200.engine.trace import TraceSession
    folder, requests, _want = model_case(tmp_models, "bitwise", cases.CASE_A, "float32", 13, [41, 18, 27])
    results = []
    for steps in (modes.whole(requests), modes.changing_portions(requests), modes.mixed(requests, live_limit=3, seed=2)):
        session = TraceSession(folder, "float32", max_tokens=modes.peak_tokens(steps), block_size=8, max_requests=3)
        got = {}
        rows = modes.expected_rows(steps)
        for s in steps:
            out = session.run_step(s)
            for r, key in enumerate(rows[s["step"]]):
                got[key] = out[r].clone()
        results.append(got)
    for other in results[1:]:
        for key in other:
            assert torch.equal(other[key], results[0][key]), f"request {key[0]} position {key[1]} differs between cuttings"


# ------------------------------------------------------------------------ far keys, page borders, the first tokens
def far_model():
    """One attention layer with sixteen heads, scores sharp enough for single keys to decide: the last heads' slopes are
    small (2^-8 for the last), so keys hundreds of tokens back still count there and nowhere else."""
    return cases.config(64, 61, [(cases.attn(16, 2, 8, 8, scale=3.0), None)], mult=1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_shows_through_the_heads_with_small_slopes(gpu, tmp_models, dtype):
    cfg = far_model()
    state = {k: v.double() for k, v in rounded(cases.seeded_state(cfg, 41), dtype).items()}
    tokens = seeded_tokens(420, cfg["vocab"], 8)
    full = plain.forward(cfg, state, tokens)
    other = list(tokens)
    other[:24] = seeded_tokens(24, cfg["vocab"], 9)           # another far past: positions 0 .. 23 only
    moved = (plain.forward(cfg, state, other) - full)[300:].abs().amax(dim=1) > 0.02 * full.abs().max()
    assert moved.sum() >= 20, "the far past does not show in these logits"
    folder = write_model_dir(str(tmp_models / f"tutizen_far_{dtype}"), cfg, {k: v.float() for k, v in state.items()}, STORED[dtype])
    requests, want = {"far": tokens}, {"far": full}
    share = 1.0 if dtype == "float32" else 0.9
    keep = {"far": set(range(0, 420, 5)) | set(range(300, 420)) | {0, 1, 2, 3, 7, 8, 9, 15, 16, 17}}
    for page in (8, 16):
        replay(folder, dtype, modes.restrict_wants(modes.whole(requests), keep), want, page, 1, "far whole", min_ok=share)
        replay(folder, dtype, modes.tail_one_by_one(requests, tail=110), want, page, 1, "far decode", min_ok=share)
        replay(folder, dtype, modes.restrict_wants(modes.changing_portions(requests, sizes=(7, 2, 64, 9, 33, 2, 120)), keep), want, page, 1,
               "far portions", min_ok=share)


def test_the_distance_penalty_is_the_designs(gpu, tmp_models):
    """The plain logits with other slopes (the exponent halved) differ outright from the design's once a few keys are in
    sight; the engine gives the design's."""
    cfg = far_model()
    state = {k: v.double() for k, v in cases.seeded_state(cfg, 43).items()}
    tokens = seeded_tokens(80, cfg["vocab"], 3)
    full = plain.forward(cfg, state, tokens)
    original = plain.head_slopes
    try:
        plain.head_slopes = lambda heads: [2.0 ** (-4.0 * (h + 1) / heads) for h in range(heads)]
        off = plain.forward(cfg, state, tokens)
    finally:
        plain.head_slopes = original
    moved = (off - full).abs().amax(dim=1) > 0.05 * full.abs().max()
    assert moved[10:].sum() >= 20
    folder = write_model_dir(str(tmp_models / "tutizen_slopes"), cfg, {k: v.float() for k, v in state.items()}, torch.float32)
    replay(folder, "float32", modes.whole({"s": tokens}), {"s": full}, 4, 1, "slopes whole")
    replay(folder, "float32", modes.tail_one_by_one({"s": tokens}, tail=50), {"s": full}, 4, 1, "slopes decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_and_long_decoding_on_the_tensor_core_sizes(gpu, tmp_models, dtype):
    """Head sizes 64 and 128 with scores five times as sharp and 120 tokens decoded one by one, across many page borders."""
    cfg = cases.sharpened(cases.CASE_C, 5.0)
    folder, requests, want = model_case(tmp_models, "sharp", cfg, dtype, 17, [389, 131])
    share = 1.0 if dtype == "float32" else 0.9
    keep = {"r0": set(range(0, 389, 7)) | set(range(260, 389)) | {0, 1, 2, 3, 15, 16, 17, 31, 32, 33, 63, 64, 65}, "r1": set(range(0, 131, 3))}
    replay(folder, dtype, modes.restrict_wants(modes.whole(requests), keep), want, 16, 2, "whole", min_ok=share)
    replay(folder, dtype, modes.restrict_wants(modes.changing_portions(requests, sizes=(7, 2, 64, 9, 33, 2, 120)), keep), want, 16, 2,
           "portions", min_ok=share)
    replay(folder, dtype, modes.tail_one_by_one(requests, tail=120), want, 16, 2, "long decode", min_ok=share)


# --------------------------------------------------------------------------- generation through the engine
def test_greedy_generation_through_the_engine(gpu, tmp_models):
    from stride_b200 import Engine, SamplingParams
    cfg = cases.CASE_A
    state = cases.seeded_state(cfg, 29)
    folder = write_model_dir(str(tmp_models / "tutizen_generate"), cfg, state, torch.float32)
    state = {k: v.double() for k, v in state.items()}
    prompts = [seeded_tokens(n, cfg["vocab"], 300 + n) for n in (37, 5, 18, 1, 26)]
    new = 9
    expected = []
    for prompt in prompts:
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(plain.forward(cfg, state, seq)[-1].argmax()))
        expected.append(seq[len(prompt):])
    # a token budget below the longest prompt: prompts go in portions beside the others' decoded tokens
    engine = Engine(folder, dtype="float32", block_size=8, num_blocks=64, max_batch_tokens=16, max_batch_seqs=3, max_model_len=64,
                    check_invariants=True)
    outs = engine.generate(copy.deepcopy(prompts), SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
    assert [o.tokens for o in outs] == expected
