"""Each mechanism of Zozenex alone on the GPU against the plain implementation: the linear-attention recurrence (a
decay per head and a gate per key channel; serial and in segments; from a state; unequal requests; the same bits under
cuts), the per-head norm with its gate, the halves rotation with rotated values and its cache write, the pooling of
blocks, attention over window and blocks with planted keys at every edge (in a portion and token by token), the
router, the grouped product of the experts, the normed branch add and the GELU."""
from types import SimpleNamespace

import pytest
import torch

import plain_zozenex as pz

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def scan_batch(lens, slots):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return SimpleNamespace(cu_q=i32(cu), slots=i32(slots), num_requests=len(lens), max_q_len=max(lens)), cu


@pytest.mark.parametrize("dtype,segment", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 4), (torch.bfloat16, 7)])
@pytest.mark.parametrize("heads,kd,vd,gated", [(2, 16, 24, False), (3, 40, 8, True), (1, 5, 70, True), (4, 32, 32, False)])
def test_linear_attention_scan_from_a_state_for_unequal_requests(dtype, segment, heads, kd, vd, gated, monkeypatch):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    monkeypatch.setattr(ops, "linear_attention_segment", segment)
    g = torch.Generator().manual_seed(2)
    lens, slots = [1, 23, 2, 70, 9], [4, 0, 5, 2, 1]      # the longest is long enough for segments
    batch, cu = scan_batch(lens, slots)
    t = cu[-1]
    # one projection buffer with q, k, v as column slices, as the mixer hands them over
    proj = torch.randn(t, 2 * heads * kd + heads * vd + 3, generator=g).to(dtype)
    state = torch.randn(6, heads, kd, vd, generator=g)
    decay = torch.rand(heads, generator=g) * 0.3 + 0.7
    z, zb, tau = torch.randn(t, heads * kd, generator=g) * 2, torch.randn(heads * kd, generator=g), 3.0
    dev = proj.to(DEV)
    q, k, v = dev[:, :heads * kd], dev[:, heads * kd:2 * heads * kd], dev[:, 2 * heads * kd:2 * heads * kd + heads * vd]
    state_dev = state.to(DEV)
    out = torch.empty(t, heads * vd, device=DEV)
    kw = {"gate": z.to(DEV), "gate_bias": zb.to(DEV), "inv_tau": 1 / tau} if gated else {"head_decay": decay.to(DEV)}
    ops.linear_attention_scan(q, k, v, heads, kd, vd, state_dev, batch, out, 0.5, 0.25, workspace=Workspace(torch.device(DEV)), **kw)
    pf = proj.double()
    for r, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        qr = pf[a:b, :heads * kd].view(-1, heads, kd) * 0.5
        kr = pf[a:b, heads * kd:2 * heads * kd].view(-1, heads, kd) * 0.25
        vr = pf[a:b, 2 * heads * kd:2 * heads * kd + heads * vd].view(-1, heads, vd)
        dec = pz.gate_decay((z[a:b] + zb).double(), tau).view(-1, heads, kd) if gated else decay.double()
        o, s_last = pz.linear_recurrence(qr, kr, vr, dec, state[slots[r]].double())
        tol = 2e-5 * max(1.0, float(o.abs().max()))
        assert float((out[a:b].cpu().double().view(-1, heads, vd) - o).abs().max()) <= tol, (r, segment)
        assert float((state_dev[slots[r]].cpu().double() - s_last).abs().max()) <= 2e-5 * max(1.0, float(s_last.abs().max())), (r, segment)
    assert torch.equal(state_dev[3].cpu(), state[3])   # a slot of no request in the step is left alone


@pytest.mark.parametrize("gated", [False, True])
def test_linear_attention_scan_in_portions_gives_the_same_bits(gated):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(3)
    heads, kd, vd, t = 2, 20, 36, 57
    q, k = torch.randn(t, heads * kd, generator=g).to(DEV), torch.randn(t, heads * kd, generator=g).to(DEV)
    v = torch.randn(t, heads * vd, generator=g).to(DEV)
    kw = {"gate": torch.randn(t, heads * kd, generator=g).to(DEV), "gate_bias": torch.randn(heads * kd, generator=g).to(DEV),
          "inv_tau": 0.25} if gated else {"head_decay": torch.tensor([0.9, 0.99]).to(DEV)}

    def run(cuts):
        state = torch.zeros(2, heads, kd, vd, device=DEV)
        out = torch.empty(t, heads * vd, device=DEV)
        for a, b in zip(cuts[:-1], cuts[1:]):
            batch = SimpleNamespace(cu_q=i32([0, b - a]), slots=i32([1]), num_requests=1, max_q_len=b - a)
            kws = dict(kw)
            if gated:
                kws["gate"] = kw["gate"][a:b]
            ops.linear_attention_scan(q[a:b], k[a:b], v[a:b], heads, kd, vd, state, batch, out[a:b], 1.0, 1.0, **kws)
        return out, state

    whole, s = run([0, t])
    for cuts in ([0, 2, 3, 30, t], list(range(t + 1))):
        o2, s2 = run(cuts)
        assert torch.equal(o2, whole) and torch.equal(s2, s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vd,weighted", [(3, 24, True), (1, 70, False), (5, 8, True)])
def test_head_norm_gate(dtype, heads, vd, weighted):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(4)
    t, eps = 13, 1e-3
    o = torch.randn(t, heads * vd, generator=g) * 3
    o[2] *= 1e-3                     # a row where eps matters
    w = torch.randn(vd, generator=g) if weighted else None
    gate = torch.randn(t, heads * vd + 5, generator=g).to(dtype)
    out = torch.empty(t, heads * vd, dtype=dtype, device=DEV)
    ops.head_norm_gate(o.to(DEV), None if w is None else w.to(DEV), gate.to(DEV)[:, 5:], heads, vd, eps, out)
    n = pz.rms_unit(o.double().view(t, heads, vd), eps)
    ref = ((n * w.double()) if weighted else n).reshape(t, heads * vd) * pz.silu(gate[:, 5:].double())
    tol = 2e-6 * 8 if dtype == torch.float32 else 2.0 ** -8 * float(ref.abs().max())
    assert float((out.cpu().double() - ref).abs().max()) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rot,rotate_values", [(6, True), (12, False), (0, True), (0, False)])
def test_halves_rotation_and_cache_write(dtype, rot, rotate_values):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.parts import half_frequencies
    g = torch.Generator().manual_seed(5)
    nq, nk, kd, vd, page = 6, 2, 12, 20, 4
    positions = [0, 1, 2, 700, 701, 5, 6, 7, 1999]
    slots = [8, 9, 10, 20, 21, 1, 2, 3, 15]
    t = len(positions)
    base = 300.0
    fk = half_frequencies(rot, base).to(DEV) if rot else None
    fv = half_frequencies(vd, base).to(DEV) if rotate_values else None
    qkv = torch.randn(t, (nq + nk) * kd + nk * vd, generator=g).to(dtype)
    kc = torch.zeros(6, nk, page, kd, dtype=dtype, device=DEV)
    vc = torch.zeros(6, nk, page, vd, dtype=dtype, device=DEV)
    dev = qkv.to(DEV)
    ops.rope_halves_kv_write(dev, i32(positions), fk, rot, fv, nq, nk, nk, kd, vd, kc, vc, i32(slots))
    src, pos = qkv.double(), torch.tensor(positions)
    q_ref = pz.rotate_halves(src[:, :nq * kd].view(t, nq, kd), pos, rot, base)
    k_ref = pz.rotate_halves(src[:, nq * kd:(nq + nk) * kd].view(t, nk, kd), pos, rot, base)
    v_ref = src[:, (nq + nk) * kd:].view(t, nk, vd)
    if rotate_values:
        v_ref = pz.rotate_halves(v_ref, pos, vd, base)
    # 32-bit angles: position * frequency carries the rounding of a 32-bit product, 2^-24 * 2,000 radians at most
    tol = 2e-3 if dtype == torch.float32 else 2.0 ** -8 * 4 + 2e-3
    got = dev.cpu().double()
    assert float((got[:, :nq * kd].view(t, nq, kd) - q_ref).abs().max()) <= tol
    assert float((got[:3, :nq * kd].view(3, nq, kd) - q_ref[:3]).abs().max()) <= (1e-6 if dtype == torch.float32 else 2.0 ** -6)
    assert torch.equal(got[:, nq * kd:], src[:, nq * kd:])            # key and value columns of the row are not rewritten
    assert torch.equal(got[:, :nq * kd].view(t, nq, kd)[..., rot:], src[:, :nq * kd].view(t, nq, kd)[..., rot:])
    for i, s in enumerate(slots):
        assert float((kc[s // page, :, s % page].cpu().double() - k_ref[i]).abs().max()) <= tol
        assert float((vc[s // page, :, s % page].cpu().double() - v_ref[i]).abs().max()) <= tol
        if not rotate_values:
            assert torch.equal(vc[s // page, :, s % page].cpu().double(), v_ref[i])
    written = torch.zeros(6 * page, dtype=torch.bool)
    written[slots] = True
    assert float(kc.float().abs().sum(dim=(1, 3)).flatten().cpu()[~written].max()) == 0.0


def planted(t, heads, kvh, kd, vd, size, pool, page, seed):
    """Queries, keys and values in which, for every query position, ONE key far outscores the rest; where it lies
    cycles through the places a fault would show: the first and last token of the window, the token right before it,
    the last token of the block seen last and the first of the block not yet seen, page borders, position 0, and a
    position hundreds back."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(t, heads, kd, generator=g) * 0.05
    k = torch.randn(t, kvh, kd, generator=g) * 0.05
    v = torch.randn(t, kvh, vd, generator=g)
    for i in range(t):
        nb = pz.visible_blocks(i, size, pool) if size and pool else 0
        lo = max(0, i - size + 1) if size else 0
        places = [lo, i, max(0, lo - 1), max(0, nb * pool - 1) if pool else 0, min(i, nb * pool) if pool else 0,
                  (i // page) * page, max(0, (i // page) * page - 1), 0, max(0, i - 300), max(0, lo - 2)]
        j = places[i % len(places)]
        d = i % kd
        for h in range(heads):
            q[i, h, d] = 6.0
        k[j, :, d] += 6.0          # several queries may plant into one key: their channels differ mostly
    return q, k, v


def paged_batch(lens_before, lens_new, page, stride=None):
    """Block tables and slot mappings for requests that hold lens_before tokens and bring lens_new more, pages dealt
    out interleaved between the requests (so that neighbours in a table are not neighbours in memory)."""
    r = len(lens_new)
    total = [a + b for a, b in zip(lens_before, lens_new)]
    rows = [n if stride is None else n // stride for n in total]
    nblk = [-(-n // page) for n in rows]
    tables, nxt = [[] for _ in range(r)], 1
    for b in range(max(nblk + [0])):
        for x in range(r):
            if b < nblk[x]:
                tables[x].append(nxt)
                nxt += 2                   # every other page stays unused (and poisoned)
    width = max(nblk + [1]) + 1
    table = torch.full((r, width), -1, dtype=torch.int32)
    for x in range(r):
        table[x, :nblk[x]] = torch.tensor(tables[x], dtype=torch.int32)
    return tables, table.to(DEV), nxt + 1


@pytest.mark.parametrize("dtype,tc", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("size,pool,page,cap,heads,kvh,kd,vd,rotv", [
    (40, 8, 16, None, 8, 2, 16, 32, True), (9, 16, 4, 5.0, 2, 2, 24, 16, False), (33, 5, 8, 20.0, 3, 1, 32, 48, True),
    (7, 3, 4, None, 6, 3, 8, 8, False), (12, None, 16, None, 2, 1, 12, 10, True), (None, None, 8, 3.0, 1, 1, 16, 6, True),
    (64, 64, 16, None, 2, 1, 64, 64, False)])
def test_window_and_block_attention_finds_the_planted_keys(dtype, tc, size, pool, page, cap, heads, kvh, kd, vd, rotv, monkeypatch):
    """Two requests of unequal length, first as one portion each (in one batch), then the last tokens of both one by
    one: rotate-and-cache, block pooling and attention run as the mixer runs them, on poisoned caches.  `tc`: the
    tensor-core kernel (for the sizes it takes; the others run on the CUDA-core kernel either way)."""
    from tiny_llm_b200 import ops
    if tc and (kd % 16 or vd % 16):
        pytest.skip("sizes the tensor-core kernel does not take")
    monkeypatch.setattr(ops, "window_attention_tc", tc)
    from tiny_llm_b200.parts import half_frequencies
    lens, tail, scale, base = [413, 150], 20, 1.0, 1000.0
    pb = torch.linspace(-9.0, -7.0, heads)       # far below zero: a key that is not planted weighs about 1e-4
    fv = half_frequencies(vd, base).to(DEV) if rotv else None
    data = [planted(n, heads, kvh, kd, vd, size, pool, page, 10 + x) for x, n in enumerate(lens)]
    quant = pz.bf16_quant if dtype == torch.bfloat16 else pz.no_quant
    refs = []
    for (q, k, v), n in zip(data, lens):
        qd, kd_, vd_ = (quant(x.double()) for x in (q, k, v))
        pos = torch.arange(n)
        vrot = quant(pz.rotate_halves(vd_, pos, vd, base)) if rotv else vd_
        o = pz.window_pool_sum(qd, kd_, vrot, scale, cap, pb.double(), size, pool, quant)
        refs.append(pz.rotate_halves(o, pos, vd, base, sign=-1.0) if rotv else o)
    # the planted keys make an edge that is off by one show: the plain result for a window one token longer differs
    # by about the size of a value row
    if size:
        (q, k, v), n = data[1], lens[1]
        other = pz.window_pool_sum(q.double(), k.double(), v.double(), scale, cap, pb.double(), size + 1, pool)
        same = pz.window_pool_sum(q.double(), k.double(), v.double(), scale, cap, pb.double(), size, pool)
        assert float((other - same).abs().max()) > 0.3

    from tiny_llm_b200.engine import Workspace
    ws = Workspace(torch.device(DEV))      # decoded tokens walk their keys in several runs that add into a buffer of it
    pages_needed = 2 * sum(-(-n // page) for n in lens) + 4
    kc = torch.full((pages_needed, kvh, page, kd), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((pages_needed, kvh, page, vd), float("nan"), dtype=dtype, device=DEV)
    pkc, pvc = torch.full_like(kc, float("nan")), torch.full_like(vc, float("nan"))
    got = [torch.zeros(n, heads, vd, dtype=torch.float64) for n in lens]

    # the tables of the final lengths, made once: a request's pages stay where they are from step to step
    tables, table, _ = paged_batch([0, 0], lens, page)
    ptables, ptable, _ = paged_batch([0, 0], lens, page, stride=pool) if pool else (None, None, None)

    def step(before, new):
        rows, posl, reql, slots, pslots = [], [], [], [], []
        for x, (a, n) in enumerate(zip(before, new)):
            q, k, v = data[x]
            for p in range(a, a + n):
                rows.append(torch.cat([q[p].flatten(), k[p].flatten(), v[p].flatten()]))
                posl.append(p)
                reql.append(x)
                slots.append(tables[x][p // page] * page + p % page)
                if pool:
                    b = p // pool
                    pslots.append(ptables[x][b // page] * page + b % page if (p + 1) % pool == 0 else -1)
        qkv = torch.stack(rows).to(dtype).to(DEV)
        cu = [0]
        for n in new:
            cu.append(cu[-1] + n)
        batch = SimpleNamespace(positions=i32(posl), token_request=i32(reql), num_tokens=len(posl), cu_q=i32(cu),
                                q_start=i32(before), num_requests=len(new), max_q_len=max(new),
                                max_kv_len=max(b + n for b, n in zip(before, new)))
        ops.rope_halves_kv_write(qkv, batch.positions, None, 0, fv, heads, kvh, kvh, kd, vd, kc, vc, i32(slots))
        if pool:
            ops.pool_kv_blocks(kc, vc, table, pkc, pvc, i32(pslots), batch, pool)
        out = torch.empty(len(posl), heads * vd, dtype=dtype, device=DEV)
        ops.window_pool_attention(qkv, heads, kvh, kd, vd, kc, vc, table, pkc if pool else None, pvc if pool else None,
                                  ptable, batch, out, scale, cap, pb.to(DEV), size, pool, fv, workspace=ws)
        o = out.cpu().double().view(-1, heads, vd)
        for row, (p, x) in enumerate(zip(posl, reql)):
            got[x][p] = o[row]

    step([0, 0], [n - tail for n in lens])
    for s in range(tail):
        step([n - tail + s for n in lens], [1, 1])
    for x, n in enumerate(lens):
        diff = (got[x] - refs[x]).abs().amax(dim=(1, 2))
        tol = 2e-4 if dtype == torch.float32 else 2.0 ** -7 * float(refs[x].abs().max())
        bad = (~(diff <= tol)).nonzero().flatten().tolist()
        assert not bad, (x, bad[:10], float(diff.max()), tol)


@pytest.mark.parametrize("experts,top,t", [(3, 3, 5), (16, 4, 300), (40, 5, 33), (7, 1, 1), (200, 8, 64)])
def test_router(experts, top, t):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(6)
    logits = torch.randn(t, experts + 3, generator=g) * 2
    corr = torch.randn(experts, generator=g)
    ids = torch.empty(t, top, dtype=torch.int32, device=DEV)
    w = torch.empty(t, top, device=DEV)
    ops.moe_route(logits.to(DEV), experts, corr.to(DEV), 2.5, ids, w)
    ref_ids, ref_w = pz.route(logits[:, :experts], corr, top, 2.5)
    assert torch.equal(ids.cpu().long(), ref_ids)            # the correction steers the choice ...
    assert float((w.cpu() - ref_w).abs().max()) <= 1e-6      # ... and stays out of the weights
    plain_choice = torch.topk(torch.sigmoid(logits[:, :experts]), top, dim=-1).indices
    assert top == experts or not torch.equal(plain_choice, ref_ids)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,t,h,ff", [(3, 3, 5, 48, 16), (16, 4, 300, 64, 40), (6, 2, 1, 96, 72), (9, 1, 130, 40, 8),
                                                  (4, 2, 450, 72, 136)])
def test_grouped_expert_products(dtype, experts, top, t, h, ff, monkeypatch):
    from tiny_llm_b200 import ops
    monkeypatch.setattr(ops, "moe_wide_tiles", True)     # tiles of 128 rows too, where an expert gets enough rows
    g = torch.Generator().manual_seed(7)
    x = torch.randn(t, h, generator=g).to(dtype)
    up, down = (torch.randn(experts, ff, h, generator=g) * 0.2).to(dtype), (torch.randn(experts, h, ff, generator=g) * 0.2).to(dtype)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(t)]).to(torch.int32)
    if t > 100:
        ids[:, 0] = 1                  # one expert gets a row of every token: several tiles
    wts = torch.rand(t, top, generator=g)
    tile = ops.moe_tile_rows(t * top, experts, tensor_cores=dtype == torch.bfloat16)
    tiles = ops.moe_max_tiles(t * top, experts, tile)
    rows = torch.empty(tiles * tile, dtype=torch.int32, device=DEV)
    texp = torch.empty(tiles, dtype=torch.int32, device=DEV)
    ops.moe_align(ids.to(DEV), experts, tile, rows, texp)
    named = rows.cpu()[rows.cpu() >= 0]
    assert sorted(named.tolist()) == list(range(t * top))          # every pair once
    for i, e in enumerate(texp.cpu().tolist()):
        members = rows.cpu()[i * tile:(i + 1) * tile]
        members = members[members >= 0]
        assert (e < 0 and len(members) == 0) or (ids.flatten()[members.long()] == e).all()
    act = torch.full((t * top, ff), float("nan"), dtype=dtype, device=DEV)
    ops.moe_linear(x.to(DEV), up.to(DEV), rows, texp, tile, act, rows_per_input=top, gelu=True)
    y = torch.full((t * top, h), float("nan"), device=DEV)
    ops.moe_linear(act, down.to(DEV), rows, texp, tile, y, rows_per_input=1, gelu=False)
    resid = torch.randn(t, h, generator=g)
    shared, logit = torch.randn(t, h, generator=g), torch.randn(t, 4, generator=g)
    out = resid.clone().to(DEV)
    ops.moe_combine(y, wts.to(DEV), shared.to(DEV), logit.to(DEV), 3, out)
    quant = pz.bf16_quant if dtype == torch.bfloat16 else pz.no_quant
    ref = resid.double()
    for i in range(t):
        for c in range(top):
            e = int(ids[i, c])
            ref[i] += wts[i, c].double() * (down[e].double() @ quant(pz.gelu_erf(up[e].double() @ x[i].double())))
        ref[i] += torch.sigmoid(logit[i, 3].double()) * shared[i].double()
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())
    assert float((out.cpu().double() - ref).abs().max()) <= tol
    out2 = resid.clone().to(DEV)
    ops.moe_combine(y, wts.to(DEV), None, None, 0, out2)       # no shared expert
    assert float((out2.cpu().double() + torch.sigmoid(logit[:, 3:4].double()) * shared.double() - ref).abs().max()) <= tol


@pytest.mark.parametrize("experts,top,t,h,ff", [(3, 3, 5, 48, 16), (16, 4, 300, 64, 40), (6, 2, 130, 96, 72), (5, 1, 700, 40, 264)])
def test_grouped_expert_products_on_tcgen05(experts, top, t, h, ff):
    """The same products through the contiguous grouped order and the tcgen05 kernel: every tile of 128 rows reads its
    own expert's rows of the stacked weights, tiles that do not exist are skipped, padding rows cost nothing."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(9)
    dtype = torch.bfloat16
    x = torch.randn(t, h, generator=g).to(dtype)
    up, down = (torch.randn(experts, ff, h, generator=g) * 0.2).to(dtype), (torch.randn(experts, h, ff, generator=g) * 0.2).to(dtype)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(t)]).to(torch.int32)
    if experts > 4:
        ids[ids == 2] = 3              # an expert that nobody chooses: its tiles do not exist
    wts = torch.rand(t, top, generator=g)
    tile = ops.MOE_TC_TILE
    tiles = ops.moe_max_tiles(t * top, experts, tile)
    rows = torch.empty(tiles * tile, dtype=torch.int32, device=DEV)
    texp = torch.empty(tiles, dtype=torch.int32, device=DEV)
    pos = torch.empty(t * top, dtype=torch.int32, device=DEV)
    ops.moe_align(ids.to(DEV), experts, tile, rows, texp, pos)
    assert torch.equal(rows.cpu()[pos.cpu().long()], torch.arange(t * top, dtype=torch.int32))
    grouped = torch.full((tiles * tile, h), float("nan"), dtype=dtype, device=DEV)
    ops.moe_gather(x.to(DEV), rows, texp, tile, grouped, rows_per_input=top)
    act = torch.full((tiles * tile, ff), float("nan"), dtype=dtype, device=DEV)
    ops.moe_linear_tc(grouped, up.to(DEV), texp, act, gelu=True)
    y = torch.full((tiles * tile, h), float("nan"), device=DEV)
    ops.moe_linear_tc(act, down.to(DEV), texp, y)
    ops.check_status()
    resid = torch.randn(t, h, generator=g)
    out = resid.clone().to(DEV)
    ops.moe_combine(y, wts.to(DEV), None, None, 0, out, pos)
    ref = resid.double()
    for i in range(t):
        for c in range(top):
            e = int(ids[i, c])
            ref[i] += wts[i, c].double() * (down[e].double() @ pz.bf16_quant(pz.gelu_erf(up[e].double() @ x[i].double())))
    assert float((out.cpu().double() - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())


def test_normed_branch_add_and_gelu():
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(8)
    for n, h in [(5, 64), (33, 200), (2, 1000), (700, 96)]:
        x, w, resid = torch.randn(n, h, generator=g) * 3, torch.randn(h, generator=g), torch.randn(n, h, generator=g)
        xd, rd = x.to(DEV), resid.clone().to(DEV)
        ops.rms_norm_add(xd, w.to(DEV), 1e-4, 0.5, rd)
        ref = resid.double() + 0.5 * pz.rms_norm(x.double(), w.double(), 1e-4)
        assert float((rd.cpu().double() - ref).abs().max()) <= 1e-5
        assert float(xd.abs().max()) == 0.0                      # the branch buffer comes back zeroed
        for dtype in (torch.float32, torch.bfloat16):
            a = x.to(dtype).to(DEV)
            ops.gelu(a, a)
            refg = pz.gelu_erf(x.to(dtype).double())
            assert float((a.cpu().double() - refg).abs().max()) <= (1e-6 if dtype == torch.float32 else 2.0 ** -8 * float(refg.abs().max()))
