"""The Zadepel design in the engine against the plain implementation of the tests: every
mechanism alone, whole prompts against decoding token by token, portions down to two tokens,
mixed batches with pages and state slots that are used again, keys far away, at page borders and
at window edges in prompts and in decoding, long decoding, and greedy generation through the
engine."""

import numpy as np
import pytest
import torch

import helpers
import plain_zadepel as plain
import zadepel_models as zm

pytestmark = pytest.mark.gpu

F32_BOUND = 2e-4          # largest |engine - plain| of a row, relative to max(1, largest |plain|)
BF16_BOUND = 6e-2
# float32 runs the sharpened weights (a key too many or too few shows); bfloat16 runs the plain
# random weights, whose rounding error stays a few percent of the logits
SHARPEN = {"float32": True, "bfloat16": False}

_folders = {}
_plain = {}


def folder_of(tmp_path_factory, name, **options):
    key = (name, tuple(sorted(options.items())))
    if key not in _folders:
        _folders[key] = zm.write_model(tmp_path_factory.mktemp(f"zadepel_{name}"), name, **options)
    return _folders[key]


def plain_rows(folder, ids):
    key = (str(folder), tuple(ids))
    if key not in _plain:
        _plain[key] = plain.logits_of(folder, ids).numpy()
    return _plain[key]


def runner_for(folder, dtype, num_pages, max_requests=4, page_size=16, **options):
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=num_pages * page_size)
    return ModelRunner(model.model, model.runtime, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests, max_step_tokens=num_pages * page_size, **options)


def assert_rows(rows, requests, folder, bound):
    """Every row within `bound` of the plain logits.  bfloat16 rounds every product's result, and
    a norm on each sublayer's output passes the relative error of a small output on at full
    size: there one row in ten may lie beyond the bound, none beyond three times it."""
    assert rows
    beyond = 0
    for (key, pos), row in sorted(rows.items()):
        want = plain_rows(folder, requests[key.split("~")[0]])[pos]
        base = max(1.0, float(np.abs(want).max()))
        diff = float(np.abs(row.astype(np.float64) - want).max())
        limit = bound * base * (3.0 if bound == BF16_BOUND else 1.0)
        assert diff <= limit, f"request {key} position {pos}: off by {diff:.3e} (bound {limit:.3e})"
        beyond += diff > bound * base
    assert beyond <= 0.1 * len(rows), f"{beyond} of {len(rows)} rows beyond the bound"


def vocab_of(name):
    return zm.CONFIGS[name]["vocab"]


# ----------------------------------------------------------------- mechanisms, kernel by kernel
def test_norms_on_both_sides_against_the_formula():
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width in (36, 256, 1000, 4104):
        delta = torch.randn(7, width, generator=g) * 3 + 0.5
        base = torch.randn(7, width, generator=g)
        gain_d, gain = torch.randn(width, generator=g), torch.randn(width, generator=g)
        for dtype in (torch.float32, torch.bfloat16):
            d = delta.to(dtype)
            summed = base.double() + plain.rms_norm(d.double(), gain_d.double(), 1e-5)
            want = plain.rms_norm(summed, gain.double(), 2e-6)
            x = base.clone().cuda()
            out = torch.empty(7, width, device="cuda", dtype=dtype)
            ops.norm_add_norm(x, d.cuda(), gain_d.cuda(), 1e-5, gain.cuda(), 2e-6, out)
            assert (x.cpu().double() - summed).abs().max() < 2e-5            # the sum stays 32-bit
            tolerance = 2e-5 if dtype is torch.float32 else 2e-2
            assert (out.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))
            # chosen rows only, x left as it is
            rows = torch.tensor([5, 0, 3], dtype=torch.int32)
            x = base.clone().cuda()
            some = torch.empty(3, width, device="cuda", dtype=dtype)
            ops.norm_add_norm(x, d.cuda(), gain_d.cuda(), 1e-5, gain.cuda(), 2e-6, some,
                              rows=rows.cuda(), write_x=False)
            assert torch.equal(x.cpu(), base)
            assert torch.equal(some, out[rows.long()])
            # the sum alone, and the norm alone
            x = base.clone().cuda()
            ops.norm_add_norm(x, d.cuda(), gain_d.cuda(), 1e-5, None, 0.0, None)
            assert (x.cpu().double() - summed).abs().max() < 2e-5
            alone = ops.norm_add_norm(base.cuda(), None, None, 0.0, gain.cuda(), 2e-6,
                                      torch.empty(7, width, device="cuda", dtype=dtype))
            want = plain.rms_norm(base.double(), gain.double(), 2e-6)
            assert (alone.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))


def test_gated_activation_against_the_formula():
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    for inter in (50, 256):
        both = torch.randn(9, 2 * inter, generator=g) * 3
        for kind, f in (("gelu_tanh", plain.gelu_tanh), ("silu", plain.silu)):
            want = f(both[:, :inter].double()) * both[:, inter:].double()
            got = ops.gated_act(both.cuda(), torch.empty(9, inter, device="cuda"), kind)
            assert (got.cpu().double() - want).abs().max() < 1e-5
            got = ops.gated_act(both.cuda().bfloat16(), torch.empty(9, inter, device="cuda", dtype=torch.bfloat16), kind)
            b = both.bfloat16().double()
            want = f(b[:, :inter]) * b[:, inter:]
            assert (got.cpu().double() - want).abs().max() < 2e-2 * float(want.abs().max())
    z = torch.tensor([-3.0, -1.0, 0.0, 0.5, 2.0], dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))


@pytest.mark.parametrize("rows,inter,k", [(300, 320, 512), (77, 100, 264), (8, 320, 512), (3, 100, 264)])
def test_products_with_the_gelu_gate_in_their_epilogue(rows, inter, k):
    """The tcgen05 products that apply the gate in their epilogue (tiles for many tokens, the
    few-token form up to 64) with the tanh form of GELU instead of SiLU."""
    import math
    from from_scratch_inference_engine_b200.kernels import ops
    torch.manual_seed(inter + rows)
    x = (torch.randn(rows, k) * 1.5).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * inter, k) / math.sqrt(k)).to(torch.bfloat16).cuda()
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    both = (x.double() @ w.double().T).to(torch.bfloat16).double()       # rounded as the unfused path
    want = plain.gelu_tanh(both[:, :inter]) * both[:, inter:]
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    if rows > 64:
        ops.gemm_tiles(ops.TiledWeight(w, swiglu=True, activation="gelu_tanh"), x, out, None, error, 148)
    else:
        ops.gemm_decode(ops.DecodeWeight(w, swiglu=True, activation="gelu_tanh"), x, out, None, error, 1)
    assert error.item() == 0
    assert (out.double() - want).abs().max().item() < 2.5e-2 * want.abs().max().item()
    unfused = ops.gated_act(both.to(torch.bfloat16).cuda(), torch.empty_like(out), "gelu_tanh")
    assert (out.double() - unfused.double()).abs().max().item() < 2.5e-2 * want.abs().max().item()


@pytest.mark.parametrize("width", [19, 128, 200])
def test_mingru_carries_state_between_calls(width):
    """Two requests of unequal length in one call, then more tokens of both in a second call (one
    of them a single token), then a long portion that runs chunk-parallel: the state left in the
    slots carries the recurrence on, a slot nobody named is untouched."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    lengths = {"a": (9, 1, 150), "b": (21, 6, 3)}
    proj = {k: torch.randn(sum(n), 3 * width, generator=g) * 2 for k, n in lengths.items()}
    state = torch.full((3, width), 7.0, device="cuda")
    state[0].zero_()
    state[2].zero_()
    slots = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    outs = {k: [] for k in lengths}
    for call in range(3):
        parts = [proj[k][sum(lengths[k][:call]):sum(lengths[k][:call + 1])] for k in ("a", "b")]
        batch = torch.cat(parts).cuda()
        qlen = torch.tensor([len(p) for p in parts], dtype=torch.int32)
        qstart = torch.tensor([0, len(parts[0])], dtype=torch.int32)
        out = torch.empty(batch.shape[0], width, device="cuda")
        chunks = {}
        if call == 2:                       # segments of 64 tokens: three of "a", one of "b"
            seg_item = torch.tensor([0, 0, 0, 1], dtype=torch.int32, device="cuda")
            seg_row0 = torch.tensor([0, 64, 128, 0], dtype=torch.int32, device="cuda")
            chunks = dict(seg_item=seg_item, seg_row0=seg_row0, num_segs=4, seg_tokens=64,
                          seg_ab=torch.empty(2 * 4 * width, device="cuda"),
                          seg_start=torch.empty(4 * width, device="cuda"))
        ops.mingru_scan(batch, width, qstart.cuda(), qlen.cuda(), slots, 2, state, out, **chunks)
        outs["a"].append(out[:len(parts[0])].cpu())
        outs["b"].append(out[len(parts[0]):].cpu())
    assert float(state[1].min()) == 7.0 and float(state[1].max()) == 7.0
    for key, slot in (("a", 2), ("b", 0)):
        p = proj[key].double()
        states = plain.mingru_states(p[:, :width], p[:, width:2 * width])
        want = states * plain.silu(p[:, 2 * width:])
        got = torch.cat(outs[key]).double()
        assert (got - want).abs().max() < 1e-5 * max(1.0, float(want.abs().max()))
        assert (state[slot].cpu().double() - states[-1]).abs().max() < 1e-5


def test_mingru_candidate_and_closed_form():
    """With a constant gate z and candidate c the state is c (1 - (1 - z)^n); the candidate is
    continuous at zero (1/2 from both sides) and grows by one per unit above it."""
    a = torch.full((40, 1), 0.3, dtype=torch.float64)
    for u0 in (-1.3, 0.0, 2.0):
        u = torch.full((40, 1), u0, dtype=torch.float64)
        z = torch.sigmoid(a[0, 0])
        cand = u0 + 0.5 if u0 >= 0 else float(torch.sigmoid(torch.tensor(u0, dtype=torch.float64)))
        want = cand * (1 - (1 - z) ** torch.arange(1, 41, dtype=torch.float64))
        assert torch.allclose(plain.mingru_states(a, u)[:, 0], want)


def _paged(rows, page_size, order, pages_total, width, dtype):
    """rows [tokens, kv_heads, width] scattered into pages [page][kv_head][slot][width] in the
    order `order` of page ids; returns (pages, block table)."""
    tokens, kv_heads, _ = rows.shape
    pages = torch.zeros(pages_total, kv_heads, page_size, width, dtype=dtype)
    table = []
    for block in range(-(-tokens // page_size)):
        page = order[block]
        table.append(page)
        chunk = rows[block * page_size:(block + 1) * page_size]
        pages[page, :, :chunk.shape[0]] = chunk.transpose(0, 1)
    return pages, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", ["small", "tensor cores"])
@pytest.mark.parametrize("window,shared", [(0, False), (37, False), (0, True), (45, True), (70, True)])
def test_scaled_attention_far_keys_page_borders_and_window_edges(dtype, window, shared, sizes):
    """Keys in shuffled pages, a request of 300 cached tokens that brings 77 more (a portion) and
    another that decodes one token at position 260, whole and split over five key ranges.  For
    chosen queries one key is made to stand out - far back, on either side of a page border, the
    last one inside the window while the first one outside it would stand out even more - so that
    reading a wrong page or slot, or a window one key off, changes the output by the size of a
    value.  `shared`: one key/value head whose values are the first columns of its key rows.
    `sizes`: key and value sizes that only the 32-bit kernel takes, or sizes that in bfloat16
    the tensor-core kernel takes as well (then both forms run)."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(5 + window)
    heads, kv_heads, page = 6, (1 if shared else 2), 16
    if sizes == "small":
        dk, dv = 24, (16 if shared else 40)
    else:
        dk, dv = (80, 64) if shared else (48, 128)
    forms = ["plain", "mma", "mma_split"] if sizes != "small" and dtype is torch.bfloat16 else ["auto"]
    group = heads // kv_heads
    lengths = [(300, 77), (260, 1)]
    pages_total = sum(-(-(a + b) // page) for a, b in lengths) + 3
    order = torch.randperm(pages_total, generator=g).tolist()
    head_scale = (0.2 + torch.rand(heads, generator=g)).double()
    k_pages = torch.zeros(pages_total, kv_heads * page * dk, dtype=dtype)
    v_pages = torch.zeros(pages_total, kv_heads * page * dv, dtype=dtype)
    tables, qs, want, used = [], [], [], 0
    for cached, new in lengths:
        n = cached + new
        k = torch.randn(n, kv_heads, dk, generator=g).to(dtype)
        q = torch.randn(new, heads, dk, generator=g)
        targets = [(new - 1, 15), (new // 2, 16), (new // 3, cached - 1), (0, 3)]
        if window:
            targets.append((new // 4, cached + new // 4 - window + 1))     # the last key inside
        for qi, kj in targets:
            q[qi] = 6.0 * k[kj, :, None, :].expand(kv_heads, group, dk).reshape(heads, dk).float() \
                / head_scale[:, None].float()
        q = q.to(dtype)
        if window:                       # the first key outside: it would win if it were seen
            outside = cached + new // 4 - window
            k[outside] = 3.0 * k[outside + 1]
        v = k[..., :dv].clone() if shared else torch.randn(n, kv_heads, dv, generator=g).to(dtype)
        blocks = -(-n // page)
        kp, table = _paged(k, page, order[used:used + blocks], pages_total, dk, dtype)
        vp, _ = _paged(v, page, order[used:used + blocks], pages_total, dv, dtype)
        used += blocks
        k_pages += kp.reshape(pages_total, -1)
        v_pages += vp.reshape(pages_total, -1)
        tables.append(table)
        qs.append(q)
        want.append(plain.windowed_attention(q.double(), k.double(), v.double(), head_scale,
                                             torch.arange(cached, n), torch.arange(n), window))
    bt = torch.full((2, max(len(t) for t in tables)), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q = torch.cat(qs).reshape(-1, heads * dk).cuda()
    tokens = q.shape[0]
    dev = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    # a page holds its keys and then, unless they live in the key rows, its values
    both = (k_pages if shared else torch.cat([k_pages, v_pages], dim=1)).cuda()
    keys = kv_heads * page * dk
    expect = torch.cat(want)
    for nsplit, form in [(n, f) for n in (1, 5) for f in forms]:
        item, row0 = [], []                    # the tiles of query rows this form of the kernel takes
        for i, (_, new) in enumerate(lengths):
            for r in range(0, new * group, ops.scaled_attention_rows(dtype, dk, dv, shared, form)):
                item.append(i)
                row0.append(r)
        out = torch.zeros(tokens, heads * dv, device="cuda", dtype=dtype)
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.scaled_attention(q, heads * dk, head_scale.float().cuda(), both[:, :keys],
                             None if shared else both[:, keys:], both.stride(0), page, dk, dv, shared,
                             bt.cuda(), dev(item), dev(row0), len(item), dev([0, 77]), dev([77, 1]),
                             dev([300, 260]), dev([0, 1]), out, tokens, heads, kv_heads, window, error,
                             nsplit, torch.empty(nsplit * tokens * heads * dv, device="cuda"),
                             torch.empty(nsplit * tokens * heads * 2, device="cuda"), form=form)
        assert int(error.item()) == 0
        got = out.cpu().double().reshape(tokens, heads, dv)
        tolerance = 2e-5 if dtype is torch.float32 else 2e-2
        assert (got - expect).abs().max() < tolerance * max(1.0, float(expect.abs().max())), (nsplit, form)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_blending_and_cache_write(dtype):
    """q rotated in place, k rotated into its page, values copied out by the first blending layer
    and blended by a later one, all at positions that differ from token to token."""
    from from_scratch_inference_engine_b200.kernels import ops
    from from_scratch_inference_engine_b200.parts.rope import rotary_table
    g = torch.Generator().manual_seed(9)
    heads, kv_heads, dim, vdim, dims, page = 4, 2, 12, 20, 8, 4
    tokens = 11
    width = (heads + kv_heads) * dim + kv_heads * vdim
    proj = torch.randn(tokens, width, generator=g).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 40, 41, 7, 100, 5, 6, 63], dtype=torch.int32)
    slot_of = torch.randperm(6 * page, generator=g)[:tokens].to(torch.int32)
    table = torch.from_numpy(rotary_table(777.0, dims, 128)).cuda()
    keys = kv_heads * page * dim
    tolerance = 1e-5 if dtype is torch.float32 else 2e-2
    first = torch.randn(tokens, kv_heads * vdim, generator=g).to(dtype)
    for mode, lam in ((0, None), (1, None), (2, 0.3)):
        pages = torch.zeros(6, keys + kv_heads * page * vdim, dtype=dtype, device="cuda")
        work = proj.clone().cuda()
        v_first = first.clone().cuda()
        mix = None if lam is None else torch.tensor([lam], device="cuda")
        ops.rotate_mix_write(work, positions.cuda(), table, slot_of.cuda(), pages[:, :keys], pages[:, keys:],
                             pages.stride(0), page, heads, kv_heads, dim, vdim, dims, mode, mix,
                             v_first if mode else None, torch.zeros(1, dtype=torch.int32, device="cuda"))
        p = proj.double()
        q = plain.rotate_half(p[:, :heads * dim].reshape(tokens, heads, dim), positions, 777.0, dims)
        k = plain.rotate_half(p[:, heads * dim:(heads + kv_heads) * dim].reshape(tokens, kv_heads, dim),
                              positions, 777.0, dims)
        v = p[:, (heads + kv_heads) * dim:].reshape(tokens, kv_heads, vdim)
        if mode == 2:
            v = (1 - lam) * v + lam * first.double().reshape(tokens, kv_heads, vdim)
        assert (work[:, :heads * dim].cpu().double().reshape(tokens, heads, dim) - q).abs().max() < tolerance * 4
        if mode == 1:
            assert torch.equal(v_first.cpu(), proj[:, (heads + kv_heads) * dim:])
        kp = pages[:, :keys].cpu().double().reshape(6, kv_heads, page, dim)
        vp = pages[:, keys:].cpu().double().reshape(6, kv_heads, page, vdim)
        for t in range(tokens):
            at = int(slot_of[t])
            assert (kp[at // page, :, at % page] - k[t]).abs().max() < tolerance * 4
            assert (vp[at // page, :, at % page] - v[t]).abs().max() < tolerance * 4


def test_rotations_keep_lengths_and_add_up():
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    positions = torch.tensor([0, 1, 2, 50, 7])
    for rotate in (plain.rotate_half, plain.rotate_interleaved):
        once = rotate(x, positions, 1000.0, 8)
        assert torch.allclose(once[..., 8:], x[..., 8:]) and torch.allclose(once[0], x[0])
        assert torch.allclose(once.norm(dim=-1), x.norm(dim=-1))
        twice = rotate(once, positions, 1000.0, 8)
        assert torch.allclose(twice, rotate(x, 2 * positions, 1000.0, 8))
    # the two layouts turn the same pairs, only stored in another order
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    half = plain.rotate_half(x[..., order + [8, 9, 10, 11]], positions, 1000.0, 8)
    inter = plain.rotate_interleaved(x, positions, 1000.0, 8)
    assert torch.allclose(half, inter[..., order + [8, 9, 10, 11]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_rows_and_products_per_head(dtype):
    """The latent is normed and the shared key part rotated into the token's cache row, the rope
    parts of the queries are rotated behind the columns that the product per head fills; and
    (U_h^T q_h) . c equals q_h . (U_h c)."""
    from from_scratch_inference_engine_b200.kernels import ops
    from from_scratch_inference_engine_b200.parts.rope import rotary_table
    g = torch.Generator().manual_seed(4)
    heads, dim, rope, rank, dims, page, tokens = 3, 10, 6, 20, 4, 4, 70
    row = rank + rope
    proj = torch.randn(tokens, heads * (dim + rope) + row, generator=g).to(dtype)
    gain = torch.randn(rank, generator=g)
    positions = torch.randint(0, 90, (tokens,), generator=g).to(torch.int32)
    slot_of = torch.randperm(20 * page, generator=g)[:tokens].to(torch.int32)
    table = torch.from_numpy(rotary_table(300.0, dims, 128)).cuda()
    pages = torch.zeros(20, page * row, dtype=dtype, device="cuda")
    qa = torch.zeros(tokens, heads * row, dtype=dtype, device="cuda")
    ops.latent_prep(proj.cuda(), positions.cuda(), table, slot_of.cuda(), pages, pages.stride(0), page,
                    gain.cuda(), 1e-5, qa, heads, dim, rope, rank, dims,
                    torch.zeros(1, dtype=torch.int32, device="cuda"))
    uk = torch.randn(heads, dim, rank, generator=g).to(dtype)             # U_h [dim, rank]
    ops.head_product(proj.cuda(), proj.shape[1], dim + rope, uk.transpose(1, 2).contiguous().cuda(), qa,
                     heads * row, row, tokens)
    tolerance = 1e-5 if dtype is torch.float32 else 2e-2
    p = proj.double()
    q = p[:, :heads * (dim + rope)].reshape(tokens, heads, dim + rope)
    lat, kr = p[:, heads * (dim + rope):heads * (dim + rope) + rank], p[:, heads * (dim + rope) + rank:]
    c = plain.rms_norm(lat, gain.double(), 1e-5)
    kr = plain.rotate_interleaved(kr, positions, 300.0, dims)
    stored = pages.cpu().double().reshape(20, page, row)
    for t in range(tokens):
        at = int(slot_of[t])
        assert (stored[at // page, at % page, :rank] - c[t]).abs().max() < tolerance * 4
        assert (stored[at // page, at % page, rank:] - kr[t]).abs().max() < tolerance * 4
    got = qa.cpu().double().reshape(tokens, heads, row)
    want_rope = plain.rotate_interleaved(q[..., dim:], positions, 300.0, dims)
    assert (got[..., rank:] - want_rope).abs().max() < tolerance * 4
    want_over = torch.einsum("thd,hdr->thr", q[..., :dim], uk.double())
    assert (got[..., :rank] - want_over).abs().max() < tolerance * max(1.0, float(want_over.abs().max()))
    # the identity behind it, in 64-bit
    k_nope = torch.einsum("hdr,tr->thd", uk.double(), c)
    assert torch.allclose(torch.einsum("thd,thd->th", q[..., :dim], k_nope),
                          torch.einsum("thr,tr->th", want_over, c))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,heads,n,k", [(70, 3, 20, 10), (9, 2, 100, 24), (1, 4, 64, 512), (16, 2, 33, 7),
                                              (150, 3, 72, 32), (300, 2, 512, 136), (64, 1, 64, 64)])
def test_product_per_head_in_its_three_forms(dtype, tokens, heads, n, k):
    """out[t, h] = W[h] x[t, h] through the kernel for few tokens, the tensor-core kernel (bfloat16,
    k in steps of 8) and the plain one; rows of x and out that lie inside wider rows."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(tokens + n)
    x_head, out_head = k + 8, n + 16
    x = torch.randn(tokens, heads * x_head, generator=g).to(dtype)
    w = (torch.randn(heads, n, k, generator=g) / k ** 0.5).to(dtype)
    out = torch.full((tokens, heads * out_head), 7.0, dtype=dtype, device="cuda")
    ops.head_product(x.cuda(), heads * x_head, x_head, w.cuda(), out, heads * out_head, out_head, tokens)
    want = torch.einsum("thk,hnk->thn", x.double().reshape(tokens, heads, x_head)[..., :k], w.double())
    got = out.cpu().double().reshape(tokens, heads, out_head)
    tolerance = 1e-5 if dtype is torch.float32 else 1e-2
    assert (got[..., :n] - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))
    assert float(got[..., n:].min()) == 7.0 and float(got[..., n:].max()) == 7.0      # nothing beyond a head's columns


def test_cache_entry_of_latent_rows():
    """A latent layer's cache entry keeps one row per token and nothing beside it; its pages go
    back behind the window."""
    from from_scratch_inference_engine_b200.cache.manager import CacheManager, CacheNeed
    need = CacheNeed(1, 26, window=10, value_dim=20, values_in_keys=True)
    assert need.v_dim == 20 and need.stored_value_dim == 0
    assert CacheNeed(2, 8, value_dim=12).stored_value_dim == 12 and CacheNeed(2, 8).stored_value_dim == 8
    cache = CacheManager([need], page_size=4, num_pages=5, num_slots=2)
    handle = cache.open("r")
    for _ in range(10):
        cache.reserve(handle, 4)
        cache.commit(handle, 4)
    assert all(page < 0 for page in handle.tables[0][:7]) and all(page >= 0 for page in handle.tables[0][7:])
    with pytest.raises(ValueError):
        need.covering(CacheNeed(1, 26, window=10, value_dim=20))


# ------------------------------------------------------------------- each mixer alone, in a model
@pytest.mark.parametrize("name", ["latent", "attention", "mingru", "odd"])
def test_one_mixer_whole_prompt_and_token_by_token(tmp_path_factory, name):
    """The prompt in one step against the same tokens one by one: the first tokens of a sequence
    (an empty state, a window that is not full yet), every window edge, page borders - as a
    prompt's rows and as decoded tokens."""
    folder = folder_of(tmp_path_factory, name)
    requests = {"p": helpers.random_ids(vocab_of(name), 70, 11)}
    runner = runner_for(folder, "float32", num_pages=8)
    rows = helpers.run_trace_in_process(runner, helpers.trace_whole(requests))
    assert len(rows) == 70
    assert_rows(rows, requests, folder, F32_BOUND)
    rows = helpers.run_trace_in_process(runner, helpers.trace_tail_by_one(requests, tail=69))
    assert len(rows) == 70
    assert_rows(rows, requests, folder, F32_BOUND)


def test_window_edge_and_blending_show_in_the_logits(tmp_path_factory):
    """The test models are sharp enough that a window one key too long or too short, a head
    without its temperature, values that are not blended or blended with the wrong layer's move
    the logits far beyond the bound that the engine is held to: the comparisons can tell."""
    folder = folder_of(tmp_path_factory, "latent")
    config, weights = plain.load(folder)
    ids = helpers.random_ids(vocab_of("latent"), 60, 11)
    right = plain.forward(config, weights, ids)
    scale = max(1.0, float(right.abs().max()))
    for size in (10, 12):
        config["layers"][0]["mixer"]["mask"] = {"size": size}
        assert float((plain.forward(config, weights, ids) - right).abs().max()) > 50 * F32_BOUND * scale
    folder = folder_of(tmp_path_factory, "attention")
    config, weights = plain.load(folder)
    ids = helpers.random_ids(vocab_of("attention"), 60, 11)
    right = plain.forward(config, weights, ids)
    scale = max(1.0, float(right.abs().max()))
    changed = dict(weights)
    changed["l2.mix.temp"] = torch.ones_like(weights["l2.mix.temp"])
    assert float((plain.forward(config, changed, ids) - right).abs().max()) > 50 * F32_BOUND * scale
    config["layers"][2]["mixer"]["v_mix"] = False
    assert float((plain.forward(config, weights, ids) - right).abs().max()) > 50 * F32_BOUND * scale
    config["layers"][2]["mixer"]["v_mix"] = True
    config["layers"][0]["mixer"]["v_mix"] = False        # layer 2 would then be the first of its kind
    assert float((plain.forward(config, weights, ids) - right).abs().max()) > 50 * F32_BOUND * scale


def test_long_prompt_runs_the_recurrence_chunk_by_chunk(tmp_path_factory):
    """A prompt long enough that the recurrence runs its chunks side by side, whole and cut in two
    inside a chunk, beside a short request in the same step; then decoding goes on from the state
    the chunks left.  The full-attention layers see keys hundreds of tokens back."""
    folder = folder_of(tmp_path_factory, "hybrid")
    requests = {"long": helpers.random_ids(vocab_of("hybrid"), 331, 3),
                "short": helpers.random_ids(vocab_of("hybrid"), 12, 4)}
    runner = runner_for(folder, "float32", num_pages=48)
    steps = [{"step": 0, "end": ["short"], "entries": [
                  {"id": "long", "tokens": requests["long"][:203], "want": [0, 63, 64, 127, 128, 202]},
                  {"id": "short", "tokens": requests["short"], "want": [11]}]},
             {"step": 1, "end": [], "entries": [
                  {"id": "long", "tokens": requests["long"][203:329], "want": [0, 60, 125]}]},
             {"step": 2, "end": [], "entries": [{"id": "long", "tokens": [requests["long"][329]], "want": [0]}]},
             {"step": 3, "end": ["long"], "entries": [{"id": "long", "tokens": [requests["long"][330]], "want": [0]}]}]
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 12
    assert_rows(rows, requests, folder, F32_BOUND)


def test_sizes_that_fit_no_vector_in_bfloat16(tmp_path_factory):
    """Width 36, feed-forward 50, vocabulary 61, head sizes 6 and 10, rank 5: no row starts on 16
    bytes.  The bfloat16 products and kernels take their plain forms; prompt, portions, decoding."""
    folder = folder_of(tmp_path_factory, "odd", sharpen=False)
    requests = {"a": helpers.random_ids(vocab_of("odd"), 45, 6), "b": helpers.random_ids(vocab_of("odd"), 19, 7)}
    runner = runner_for(folder, "bfloat16", num_pages=8)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=1, max_live=2)):
        rows = helpers.run_trace_in_process(runner, steps)
        assert len(rows) == 64
        assert_rows(rows, requests, folder, BF16_BOUND)


# ---------------------------------------------------------------------------- the whole design
@pytest.mark.parametrize("name", ["hybrid", "wide"])
@pytest.mark.parametrize("dtype,bound", [("float32", F32_BOUND), ("bfloat16", BF16_BOUND)])
def test_portions_of_every_size(tmp_path_factory, name, dtype, bound):
    folder = folder_of(tmp_path_factory, name, sharpen=SHARPEN[dtype])
    requests = {"a": helpers.random_ids(vocab_of(name), 90, 1),
                "b": helpers.random_ids(vocab_of(name), 37, 2)}
    runner = runner_for(folder, dtype, num_pages=8)
    steps = helpers.trace_portions(requests, seed=3)
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) <= 2
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 127
    assert_rows(rows, requests, folder, bound)


@pytest.mark.parametrize("dtype,bound", [("float32", F32_BOUND), ("bfloat16", BF16_BOUND)])
def test_mixed_batches_reuse_pages_and_slots(tmp_path_factory, dtype, bound):
    """Six unequal requests through two state slots and a pool that holds little more than two of
    them: portions of one beside single tokens of another, requests that sit a step out, one
    that is released in the middle and fed again from its first token - every request's rows
    equal what it gives alone."""
    folder = folder_of(tmp_path_factory, "hybrid", sharpen=SHARPEN[dtype])
    lengths = {"a": 75, "b": 9, "c": 41, "d": 1, "e": 58, "f": 26}
    requests = {k: helpers.random_ids(vocab_of("hybrid"), n, i + 20)
                for i, (k, n) in enumerate(lengths.items())}
    steps, names = helpers.trace_mixed_with_recompute(requests, seed=5, max_live=2)
    need = helpers.live_tokens_needed(steps, round_to=16)
    runner = runner_for(folder, dtype, num_pages=need // 16, max_requests=2)
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) >= sum(lengths.values())
    assert_rows(rows, names, folder, bound)
    assert runner.cache.slots.num_free == 2
    assert all(free == need // 16 for free in runner.cache.free_pages())


def test_long_decoding_through_graphs_and_without(tmp_path_factory):
    """A short prompt, then 150 tokens one by one: the window passes over decoded tokens, pages
    are given back on the way, and the decode steps replay captured graphs; the same without
    graphs gives the same rows up to the order of the sums (a captured step cuts the keys into
    ranges by the longest context its block tables can hold, not by the context it meets)."""
    folder = folder_of(tmp_path_factory, "hybrid")
    requests = {"long": helpers.random_ids(vocab_of("hybrid"), 157, 9)}
    steps = helpers.trace_tail_by_one(requests, tail=150)
    both = []
    for graphs in (True, False):
        runner = runner_for(folder, "float32", num_pages=12, cuda_graphs=graphs)
        assert runner.cuda_graphs == graphs
        rows = helpers.run_trace_in_process(runner, steps)
        assert_rows(rows, requests, folder, F32_BOUND)
        both.append(rows)
    for key in both[0]:
        assert float(np.abs(both[0][key] - both[1][key]).max()) < 0.25 * F32_BOUND


def test_decode_batch_with_padding_leaves_other_slots_alone(tmp_path_factory):
    """Three requests decode together in a captured batch of four: the padding entry must not
    touch the state of slot 0, which a live request holds, nor any page."""
    folder = folder_of(tmp_path_factory, "hybrid")
    requests = {k: helpers.random_ids(vocab_of("hybrid"), n, s)
                for k, n, s in (("a", 30, 1), ("b", 22, 2), ("c", 26, 3))}
    runner = runner_for(folder, "float32", num_pages=12)
    steps = [{"step": 0, "end": [], "entries": [
        {"id": k, "tokens": ids[:12], "want": [11]} for k, ids in requests.items()]}]
    for t in range(12, 22):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": k, "tokens": [ids[t]], "want": [0]} for k, ids in requests.items()]})
    steps[-1]["end"] = list(requests)
    rows = helpers.run_trace_in_process(runner, steps)
    assert runner._graphs
    assert_rows(rows, requests, folder, F32_BOUND)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path_factory, dtype):
    """Requests of unequal length through `Engine` and its scheduler with a small token budget
    (prompts go in portions) and two slots: every generated token is the plain implementation's
    choice; where the plain logits are a near tie the engine may pick either."""
    from from_scratch_inference_engine_b200 import Engine, LoadedModel, SamplingParams
    folder = folder_of(tmp_path_factory, "hybrid", sharpen=SHARPEN[dtype])
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=256)
    engine = Engine(model, block_size=16, num_blocks=16, max_batch=2, max_step_tokens=24)
    prompts = [helpers.random_ids(vocab_of("hybrid"), n, s) for n, s in ((45, 1), (7, 2), (30, 3))]
    ids = [engine.add_request(p, SamplingParams(temperature=0.0), 8) for p in prompts]
    engine.run_until_done()
    config, weights = plain.load(folder)
    slack = 1e-3 if dtype == "float32" else 0.15
    for rid, prompt in zip(ids, prompts):
        seq = list(prompt)
        assert len(engine.output(rid)) == 8
        for token in engine.output(rid):
            logits = plain.forward(config, weights, seq)[-1]
            assert float(logits.max() - logits[token]) <= slack * max(1.0, float(logits.abs().max()))
            seq.append(token)


def test_llm_entry_point_reads_the_design_by_its_name(tmp_path_factory):
    from from_scratch_inference_engine_b200 import LLM, GenerationConfig, load_config
    folder = folder_of(tmp_path_factory, "odd")
    assert type(load_config(folder)).__name__ == "ZadepelConfig"
    llm = LLM(folder, block_size=16, num_blocks=8, max_batch=2, dtype="float32", eos_id=-1)
    prompt = helpers.random_ids(vocab_of("odd"), 19, 4)
    got = llm.generate_ids(prompt, GenerationConfig(max_tokens=5))
    assert len(got) == 5
    config, weights = plain.load(folder)
    seq = list(prompt)
    for token in got:
        logits = plain.forward(config, weights, seq)[-1]
        assert float(logits.max() - logits[token]) <= 1e-3 * max(1.0, float(logits.abs().max()))
        seq.append(token)


@pytest.mark.parametrize("dtype,name,bound", [("float32", "hybrid", F32_BOUND), ("bfloat16", "wide", BF16_BOUND)])
def test_trace_replay_program_runs_the_design(tmp_path_factory, tmp_path, dtype, name, bound):
    """bin/trace_run as a user runs it (a subprocess, steps on standard input, logits in files)
    on a mixed trace of five requests through four slots and a pool for the live tokens only."""
    import json
    import subprocess
    from pathlib import Path
    folder = folder_of(tmp_path_factory, name, sharpen=SHARPEN[dtype])
    vocab = vocab_of(name)
    requests = {key: helpers.random_ids(vocab, n, i)
                for i, (key, n) in enumerate({"a": 90, "b": 40, "c": 70, "d": 33, "e": 64}.items())}
    steps = helpers.trace_mixed(requests, seed=3)
    need = helpers.live_tokens_needed(steps, round_to=64)
    root = Path(__file__).resolve().parent.parent
    text = "".join(json.dumps(step) + "\n" for step in steps)
    done = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(tmp_path / "out"), "--max-tokens", str(need)],
                          input=text, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: np.fromfile(tmp_path / "out" / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
               for s in steps if any(e["want"] for e in s["entries"])}
    rows = helpers.collect_rows(steps, outputs)
    assert len(rows) == sum(len(ids) for ids in requests.values())
    assert_rows(rows, requests, folder, bound)
