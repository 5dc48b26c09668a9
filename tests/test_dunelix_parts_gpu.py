"""Each new mechanism alone on the GPU against the plain implementation: Dynamic Tanh, the minGRU recurrence (walked
serially and in segments, from a state, for unequal requests), the pairwise rotation with its cache write, attention
with two score maps over paged keys (chunk edges, page borders, far keys, in a portion and for a single token), and
the differential combine."""
from types import SimpleNamespace

import pytest
import torch

import plain_dunelix as pd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(1)
    for n, h in [(5, 64), (33, 200), (2, 1000), (3, 50), (2500, 96)]:
        x = torch.randn(n, h, generator=g) * 3
        w, b, alpha = torch.randn(h, generator=g), torch.randn(h, generator=g), torch.tensor([0.37])
        out = torch.empty(n, h, dtype=dtype, device=DEV)
        ops.dyt_norm(x.to(DEV), w.to(DEV), b.to(DEV), alpha.to(DEV), out)
        ref = pd.dynamic_tanh(x, w, b, alpha)
        tol = 2e-6 if dtype == torch.float32 else 2.0 ** -8 * float(ref.abs().max())
        assert float((out.float().cpu() - ref).abs().max()) <= tol
        rows = [n - 1, 0]
        out2 = torch.empty(2, h, dtype=dtype, device=DEV)
        ops.dyt_norm(x.to(DEV), w.to(DEV), b.to(DEV), alpha.to(DEV), out2, i32(rows))
        assert torch.equal(out2, out[rows])


def scan_batch(lens):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return SimpleNamespace(cu_q=i32(cu), slots=None, num_requests=len(lens), max_q_len=max(lens)), cu


@pytest.mark.parametrize("dtype,segment", [(torch.float32, 0), (torch.bfloat16, 0), (torch.bfloat16, 4), (torch.bfloat16, 5)])
def test_min_gru_scan_from_a_state_for_unequal_requests(dtype, segment, monkeypatch):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    monkeypatch.setattr(ops, "min_gru_segment", segment)
    g = torch.Generator().manual_seed(2)
    width, lens, slots = 70, [1, 23, 2, 40, 9], [4, 0, 5, 2, 1]
    batch, cu = scan_batch(lens)
    batch.slots = i32(slots)
    t = cu[-1]
    zug = (torch.randn(t, 3 * width, generator=g) * 2).to(dtype)
    bz, bu = torch.randn(width, generator=g), torch.randn(width, generator=g)
    state = torch.rand(6, width, generator=g)
    state_dev = state.to(DEV)
    out = torch.empty(t, width, dtype=dtype, device=DEV)
    ops.min_gru_scan(zug.to(DEV), bz.to(DEV), bu.to(DEV), state_dev, batch, out, Workspace(torch.device(DEV)))
    zf = zug.float()
    for r, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        z = torch.sigmoid(zf[a:b, :width] + bz)
        cand = pd.min_gru_candidate(zf[a:b, width:2 * width] + bu)
        s_all, s_last = pd.min_gru_scan(z, cand, state[slots[r]])
        y = s_all * pd.silu(zf[a:b, 2 * width:])
        tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8 * float(y.abs().max())
        assert float((out[a:b].float().cpu() - y).abs().max()) <= tol, (r, segment)
        assert float((state_dev[slots[r]].cpu() - s_last).abs().max()) <= 1e-5, (r, segment)
    assert torch.equal(state_dev[3].cpu(), state[3])   # a slot of no request in the step is left alone


def test_min_gru_scan_in_portions_gives_the_same_bits():
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(3)
    width, t = 33, 57
    zug = torch.randn(t, 3 * width, generator=g).to(DEV)
    bz, bu = torch.randn(width, generator=g).to(DEV), torch.randn(width, generator=g).to(DEV)

    def run(cuts):
        state = torch.zeros(2, width, device=DEV)
        out = torch.empty(t, width, device=DEV)
        for a, b in zip(cuts[:-1], cuts[1:]):
            batch = SimpleNamespace(cu_q=i32([0, b - a]), slots=i32([1]), num_requests=1, max_q_len=b - a)
            ops.min_gru_scan(zug[a:b], bz, bu, state, batch, out[a:b])
        return out, state

    whole, s = run([0, t])
    for cuts in ([0, 2, 3, 30, t], list(range(t + 1))):
        o2, s2 = run(cuts)
        assert torch.equal(o2, whole) and torch.equal(s2, s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pairwise_rotation_and_cache_write(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(4)
    nq, nk, nv, kd, vd, page, rot = 6, 4, 2, 12, 20, 4, 6
    t = 9
    positions = [0, 1, 2, 700, 701, 5, 6, 7, 31999]
    slots = [8, 9, 10, 20, 21, 1, 2, 3, 15]
    freq = pd.scaled_frequencies(rot, 50.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
    qkv = torch.randn(t, (nq + nk) * kd + nv * vd, generator=g).to(dtype)
    kc = torch.zeros(6, nk, page, kd, dtype=dtype, device=DEV)
    vc = torch.zeros(6, nv, page, vd, dtype=dtype, device=DEV)
    dev = qkv.to(DEV)
    ops.rope_pairs_kv_write(dev, i32(positions), freq.to(DEV), rot, nq, nk, nv, kd, vd, kc, vc, i32(slots))
    src = qkv.float()
    pos = torch.tensor(positions)
    q_ref = pd.rotate_interleaved(src[:, :nq * kd].view(t, nq, kd), pos, freq)
    k_ref = pd.rotate_interleaved(src[:, nq * kd:(nq + nk) * kd].view(t, nk, kd), pos, freq)
    v_ref = src[:, (nq + nk) * kd:].view(t, nv, vd)
    tol = 2e-6 * 4 if dtype == torch.float32 else 2.0 ** -8 * 4
    got = dev.float().cpu()
    assert float((got[:, :nq * kd].view(t, nq, kd) - q_ref).abs().max()) <= tol
    assert torch.equal(got[:, nq * kd:], src[:, nq * kd:])            # key and value columns of the row are not rewritten
    assert torch.equal(q_ref[..., rot:], src[:, :nq * kd].view(t, nq, kd)[..., rot:])   # the tail of a row passes unchanged
    for i, s in enumerate(slots):
        assert float((kc[s // page, :, s % page].float().cpu() - k_ref[i]).abs().max()) <= tol
        assert torch.equal(vc[s // page, :, s % page].float().cpu(), v_ref[i])
    written = torch.zeros(6 * page, dtype=torch.bool)
    written[slots] = True
    assert float(kc.float().abs().sum(dim=(1, 3)).flatten().cpu()[~written].max()) == 0.0


def paged(rows, table, page, pages):
    """rows [T, heads, d] -> cache [pages, heads, page, d] with position j in page table[j // page]."""
    t, heads, d = rows.shape
    cache = torch.full((pages, heads, page, d), float("nan"), dtype=rows.dtype)
    for j in range(t):
        cache[table[j // page], :, j % page] = rows[j]
    return cache


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk,page,length", [(None, 16, 700), (180, 16, 620), (24, 8, 100), (7, 4, 50)])
def test_attention_maps_sees_exactly_the_chunk_and_finds_a_planted_key(dtype, chunk, page, length):
    """Keys are small but for one planted key per query position whose score stands out; it lies far back, at a page
    border, on the first position of the query's chunk (visible) or right before it (not visible).  Whether the
    kernel followed it shows in the output, which is then that key's value row or not."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(5)
    heads, kvh, maps, kd, vd = 4, 2, 2, 16, 24
    group = heads // kvh
    k = torch.randn(length, kvh * maps, kd, generator=g) * 0.05
    v = torch.randn(length, kvh, vd, generator=g)
    pages_needed = -(-length // page)
    table = torch.randperm(pages_needed + 3, generator=g)[:pages_needed].tolist()
    # query positions: the last one, chunk edges, page edges
    qpos = sorted({length - 1, 0, 1, page - 1, page, length // 2} |
                  ({(length // chunk) * chunk - 1, (length // chunk) * chunk, chunk - 1, chunk} if chunk else set()))
    qpos = [p for p in qpos if 0 <= p < length]
    plants = {}
    q = torch.randn(len(qpos), heads * maps, kd, generator=g) * 0.05
    for i, p in enumerate(qpos):
        start = (p // chunk) * chunk if chunk else 0
        inside = [start, (p // page) * page, max(start, p - 3)]
        outside = [start - 1] if start > 0 else []
        target = (inside + outside)[(i + 1) % (len(inside) + len(outside))]
        plants[p] = target
        direction = torch.zeros(kd)
        direction[i] = 1.0     # one axis per query position: a key planted for one query says nothing to another
        for m in range(maps):
            k[target, 0 * maps + m] += 6.0 * direction * (1 if m == 0 else -1)
            for h in range(group):
                q[i, (0 * group + h) * maps + m] += 6.0 * direction * (1 if m == 0 else -1)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 1.7
    kc, vc = paged(k, table, page, pages_needed + 3).to(DEV), paged(v, table, page, pages_needed + 3).to(DEV)
    bt = i32([table + [-1] * 5])
    ref = torch.empty(len(qpos), heads * maps, vd)
    kp = torch.arange(length)
    for i, p in enumerate(qpos):
        mask = pd.chunk_mask(torch.tensor([p]), kp, chunk) if chunk else (kp[None, :] <= p)
        for h in range(heads):
            for m in range(maps):
                ref[i, h * maps + m] = pd.softmax_attention(q[i:i + 1, h * maps + m].float(), k[:, (h // group) * maps + m].float(),
                                                            v[:, h // group].float(), mask, scale)[0]
    # the planted key decides the output of head 0 exactly when it is visible
    for i, p in enumerate(qpos):
        visible = plants[p] <= p and (not chunk or plants[p] // chunk == p // chunk)
        close = float((ref[i, 0] - v[plants[p], 0].float()).abs().max()) < 0.05
        assert close == visible or plants[p] > p, (p, plants[p])
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())

    def run(rows, out_dtype, generic=False):
        """Every query position a request of its own with one token (as decoded tokens run), all on the same pages."""
        n = len(rows)
        positions = [qpos[i] for i in rows]
        batch = SimpleNamespace(token_request=i32(list(range(n))), positions=i32(positions), cu_q=i32(list(range(n + 1))),
                                q_start=i32(positions), num_requests=n, max_q_len=1)
        qrows = q[rows].reshape(n, -1)
        pad = torch.zeros(n, 40, dtype=dtype)     # the queries lie at the front of wider rows
        out = torch.empty(n, heads * maps * vd, dtype=out_dtype, device=DEV)
        ops.force_generic = generic
        try:
            ops.paged_attention_maps(torch.cat([qrows, pad], dim=1).to(DEV), heads, kvh, maps, kd, vd, kc, vc,
                                     bt.repeat(n, 1).contiguous(), batch, out, scale, None, chunk)
        finally:
            ops.force_generic = False
        return out.float().cpu().view(n, heads * maps, vd)

    everyone = list(range(len(qpos)))
    for generic in (True, False):      # the CUDA-core kernel, then (bfloat16 only) the tensor-core kernel
        together = run(everyone, torch.float32, generic)
        assert torch.isfinite(together).all()
        assert float((together - ref).abs().max()) <= tol, generic
        for i, p in enumerate(qpos):       # every position alone: another launch shape
            alone = run([i], torch.float32, generic)
            assert float((alone[0] - ref[i]).abs().max()) <= tol, (p, generic)
            if dtype == torch.float32:
                assert torch.equal(alone[0], together[i]), p
    if dtype == torch.bfloat16:
        same_type = run(everyone, torch.bfloat16)
        assert float((same_type - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kd,vd,heads,kvh,chunk,page", [(16, 32, 4, 2, 24, 8), (48, 80, 6, 3, 150, 16), (64, 128, 6, 1, None, 16),
                                                        (32, 16, 2, 2, 7, 4), (24, 40, 3, 3, 50, 16)])
def test_attention_maps_portions_of_unequal_requests(dtype, kd, vd, heads, kvh, chunk, page):
    """Three requests in one step: a portion that starts inside a chunk and crosses chunk and page edges, a single
    decoded token, and a prompt from position 0; both kernels against the plain implementation."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(kd + vd)
    maps, group = 2, heads // kvh
    spans = [(130, 97), (211, 1), (0, 75)]                 # (first position, tokens) of each request in this step
    lengths = [a + n for a, n in spans]
    scale = 0.9
    caches, tables, next_page = [], [], 0
    total_pages = sum(-(-n // page) for n in lengths) + 2
    kc = torch.full((total_pages, kvh * maps, page, kd), float("nan"), dtype=dtype)
    vc = torch.full((total_pages, kvh, page, vd), float("nan"), dtype=dtype)
    order = torch.randperm(total_pages, generator=g).tolist()
    ks, vs = [], []
    for n in lengths:
        k = (torch.randn(n, kvh * maps, kd, generator=g) * 0.7).to(dtype)
        v = torch.randn(n, kvh, vd, generator=g).to(dtype)
        table = [order.pop() for _ in range(-(-n // page))]
        for j in range(n):
            kc[table[j // page], :, j % page] = k[j]
            vc[table[j // page], :, j % page] = v[j]
        ks.append(k), vs.append(v), tables.append(table)
    width = max(len(t) for t in tables) + 2
    bt = i32([t + [-1] * (width - len(t)) for t in tables])
    t_all = sum(n for _, n in spans)
    q = (torch.randn(t_all, heads * maps, kd, generator=g) * 0.7).to(dtype)
    ref = torch.empty(t_all, heads * maps, vd)
    row = 0
    cu, req_of, pos_of = [0], [], []
    for r, (a, n) in enumerate(spans):
        qp, kp = torch.arange(a, a + n), torch.arange(lengths[r])
        mask = pd.chunk_mask(qp, kp, chunk) if chunk else (kp[None, :] <= qp[:, None])
        for h in range(heads):
            for m in range(maps):
                ref[row:row + n, h * maps + m] = pd.softmax_attention(q[row:row + n, h * maps + m].float(),
                                                                      ks[r][:, (h // group) * maps + m].float(),
                                                                      vs[r][:, h // group].float(), mask, scale)
        row += n
        cu.append(row)
        req_of += [r] * n
        pos_of += list(range(a, a + n))
    batch = SimpleNamespace(token_request=i32(req_of), positions=i32(pos_of), cu_q=i32(cu), q_start=i32([a for a, _ in spans]),
                            num_requests=len(spans), max_q_len=max(n for _, n in spans))
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())
    for generic in (True, False):
        out = torch.empty(t_all, heads * maps * vd, dtype=torch.float32, device=DEV)
        ops.force_generic = generic
        try:
            ops.paged_attention_maps(q.reshape(t_all, -1).to(DEV), heads, kvh, maps, kd, vd, kc.to(DEV), vc.to(DEV), bt, batch,
                                     out, scale, None, chunk)
        finally:
            ops.force_generic = False
        got = out.cpu().view(t_all, heads * maps, vd)
        assert torch.isfinite(got).all(), generic
        bad = ((got - ref).abs().amax(dim=(1, 2)) > tol).nonzero().flatten().tolist()
        assert not bad, (generic, [(req_of[i], pos_of[i]) for i in bad[:8]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_differential_combine(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(6)
    for t, heads, vd, kd, diff, eps in [(7, 3, 40, 16, 0.3, 1e-5), (130, 2, 96, 48, 0.5, 1e-6), (1, 5, 7, 10, 0.8, 1e-3)]:
        a = torch.randn(t, heads, 2, vd, generator=g)
        lam_w = [torch.randn(kd, generator=g) * 0.4 for _ in range(4)]
        out = torch.empty(t, heads * vd, dtype=dtype, device=DEV)
        ops.diff_combine(a.to(DEV), *[x.to(DEV) for x in lam_w], diff, eps, out)
        lam = pd.differential_lambda(*lam_w, diff)
        o = a[:, :, 0] - lam * a[:, :, 1]
        ref = (o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps) * (1.0 - diff)).reshape(t, heads * vd)
        tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8 * float(ref.abs().max())
        assert float((out.float().cpu() - ref).abs().max()) <= tol


@pytest.mark.parametrize("m,n,k", [(8, 768, 1024), (3, 1000, 2048), (64, 6144, 512)])
def test_input_projection_of_few_rows_with_k_slices_in_a_cluster(m, n, k):
    """What the mixers' input projections ask for at decode: a bfloat16 product of few rows whose K slices meet in a
    thread-block cluster (one writer per element: two runs give the same bits)."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(9)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    assert ops._cluster_slices(n, k) > 1
    ref = a.double() @ w.double().T
    outs = []
    for _ in range(2):
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        ops.linear(a.to(DEV), w.to(DEV), out, cluster_slices=True)
        outs.append(out.float().cpu())
    assert float((outs[0] - ref.float()).abs().max()) <= 2.0 ** -8 * float(ref.abs().max())
    assert torch.equal(outs[0], outs[1])
    ops.check_status()
