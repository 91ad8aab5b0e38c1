"""Each CUDA kernel alone against a plain torch formula, at sizes other than the models'.

Error measure as in the reference's kernel tests (bench/test_kernels.py:18-33): largest
absolute error over the reference tensor's largest magnitude; 2e-2 for bfloat16 storage,
1e-5 for 32-bit.
"""

import math

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}
DTYPES = [torch.float32, torch.bfloat16]


def K():
    from enginekernel_b200.ops import kernels
    return kernels


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-9)


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------ norms, embedding, gate
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(1, 80), (37, 2560), (5, 1000), (3, 12288)])
def test_rmsnorm_plain_add_and_gathered(dtype, rows, hidden):
    k = K()
    stream = rnd(rows, hidden, seed=1)
    gain = 1 + 0.1 * rnd(hidden, seed=2)
    add = rnd(rows, hidden, dtype=dtype, seed=3)
    eps = 3e-6

    def ref(x):
        x = x.double()
        return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain.double())

    y = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    k.rmsnorm(y, stream.clone(), gain, eps)
    assert rel(y, ref(stream)) <= TOL[dtype]

    s2 = stream.clone()
    k.rmsnorm(y, s2, gain, eps, add=add)
    summed = stream.double() + add.double()
    assert rel(s2, summed) <= 1e-6                       # the stream itself stays 32-bit
    assert rel(y, ref(summed)) <= TOL[dtype]

    pick = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device=DEV)
    s3 = stream.clone()
    y3 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    k.rmsnorm(y3, s3, gain, eps, add=add, rows=pick, write_back=False)
    assert torch.equal(s3, stream)                       # not written back
    assert rel(y3, ref(summed)[pick.long().cpu()]) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_and_silu_mul(dtype):
    k = K()
    table = rnd(331, 80, dtype=dtype, seed=4)
    ids = torch.tensor([0, 330, 7, 7, 100], dtype=torch.int32, device=DEV)
    out = torch.zeros(6, 80, device=DEV)
    k.embed(out, table, ids, 5)
    assert torch.equal(out[:5], table[ids.long()].float()) and out[5].abs().sum() == 0

    for rows, inter in ((1, 176), (19, 9728), (4, 1001), (3, 1004)):
        gu = rnd(rows, 2 * inter, dtype=dtype, seed=5, scale=2.0)
        act = torch.empty(rows, inter, dtype=dtype, device=DEV)
        k.silu_mul(act, gu)
        g, u = gu.double()[:, :inter], gu.double()[:, inter:]
        assert rel(act, g / (1 + torch.exp(-g)) * u) <= TOL[dtype]


# ------------------------------------------------------------------ paged cache helpers
class Pages:
    """A little paged cache with a shuffled page order, plus its dense mirror."""

    def __init__(self, n_slots, max_len, heads, d, dtype, seed=0):
        self.page = K().PAGE
        per = -(-max_len // self.page)
        n_pages = n_slots * per + 3
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(n_pages, generator=g)[: n_slots * per].view(n_slots, per)
        self.table = perm.to(torch.int32).to(DEV)
        self.k = torch.zeros(n_pages, heads, self.page, d, dtype=dtype, device=DEV)
        self.v = torch.zeros_like(self.k)
        self.heads, self.d = heads, d

    def fill(self, slot, keys, values):
        """keys/values [len, heads, d] written at positions 0..len-1 of ``slot``."""
        for p in range(keys.shape[0]):
            page = int(self.table[slot, p // self.page])
            self.k[page, :, p % self.page] = keys[p]
            self.v[page, :, p % self.page] = values[p]

    def dense(self, slot, length):
        idx = torch.arange(length)
        pages = self.table[slot, (idx // self.page).to(DEV)].long()
        off = (idx % self.page).to(DEV)
        return self.k[pages, :, off], self.v[pages, :, off]      # [len, heads, d]


def ref_attention(q, keys, values, pos, scale, window=None):
    """q [NH, D] at position pos over keys/values [len, NKV, D] (len > pos), float64."""
    nh, nkv = q.shape[0], keys.shape[1]
    lo = 0 if not window else max(0, pos - window + 1)
    kk = keys[lo:pos + 1].double().repeat_interleave(nh // nkv, 1)
    vv = values[lo:pos + 1].double().repeat_interleave(nh // nkv, 1)
    s = torch.einsum("hd,jhd->hj", q.double(), kk) * scale
    p = torch.softmax(s, -1)
    return torch.einsum("hj,jhd->hd", p, vv).reshape(-1)


# ------------------------------------------------------------------ rope + cache write
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot", [(4, 2, 16, 16), (6, 3, 48, 48), (8, 1, 128, 128),
                                          (2, 2, 80, 32), (3, 1, 256, 256)])
def test_qk_norm_rope_kv(dtype, nq, nkv, d, rot):
    k = K()
    eps, theta, max_len, n_slots = 1e-5, 50000.0, 200, 3
    pages = Pages(n_slots, max_len, nkv, d, dtype, seed=d)
    before_k, before_v = pages.k.clone(), pages.v.clone()
    toks = [(0, 0), (0, 1), (2, 63), (2, 64), (1, 199), (1, -1), (0, 130)]     # (slot, position)
    t = len(toks)
    qkv = rnd(t, (nq + 2 * nkv) * d, dtype=dtype, seed=7)
    orig = qkv.clone()
    qg, kg = 1 + 0.1 * rnd(d, seed=8), 1 + 0.1 * rnd(d, seed=9)
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    freqs = torch.outer(torch.arange(max_len, dtype=torch.float32), inv)
    cos, sin = freqs.cos().to(DEV), freqs.sin().to(DEV)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    k.qk_norm_rope_kv(qkv, t, qg, kg, cos, sin, rot, positions, slots, pages.k, pages.v,
                      pages.table, nq, nkv, d, eps)

    def ref_head(x, gain, p):
        x = x.double()
        x = x * torch.rsqrt(x.pow(2).mean() + eps) * gain.double().cpu()
        out = x.clone()
        h = rot // 2
        c, s = freqs[p].cos().double(), freqs[p].sin().double()
        out[:h] = x[:h] * c - x[h:rot] * s
        out[h:rot] = x[h:rot] * c + x[:h] * s
        return out

    touched = set()
    for i, (slot, p) in enumerate(toks):
        row = orig[i].cpu()
        if p < 0:                                        # a finished row: nothing happens
            assert torch.equal(qkv[i], orig[i])
            continue
        for h in range(nq):
            want = ref_head(row[h * d:(h + 1) * d], qg, p)
            assert rel(qkv[i, h * d:(h + 1) * d], want) <= TOL[dtype]
        page = int(pages.table[slot, p // 64])
        for h in range(nkv):
            want = ref_head(row[(nq + h) * d:(nq + h + 1) * d], kg, p)
            assert rel(pages.k[page, h, p % 64], want) <= TOL[dtype]
            assert torch.equal(pages.v[page, h, p % 64], orig[i, (nq + nkv + h) * d:(nq + nkv + h + 1) * d])
            touched.add((page, h, p % 64))
    # everything else in the cache is untouched
    mask = torch.ones(pages.k.shape[:3], dtype=torch.bool)
    for page, h, o in touched:
        mask[page, h, o] = False
    assert torch.equal(pages.k.cpu()[mask], before_k.cpu()[mask])
    assert torch.equal(pages.v.cpu()[mask], before_v.cpu()[mask])
    # a run that must not write the cache leaves it alone but still rotates q
    k2, v2, q2 = pages.k.clone(), pages.v.clone(), orig.clone()
    k.qk_norm_rope_kv(q2, t, qg, kg, cos, sin, rot, positions, slots, k2, v2, pages.table, nq, nkv,
                      d, eps, write_kv=False)
    assert torch.equal(k2, pages.k) and torch.equal(v2, pages.v)
    assert torch.equal(q2[:, :nq * d], qkv[:, :nq * d])


@pytest.mark.parametrize("per_slot", [100, 250])
@pytest.mark.parametrize("nq,nkv,d,gains", [(5, 1, 64, True), (120, 8, 64, True), (12, 3, 128, True),
                                            (60, 4, 128, False), (3, 2, 256, True), (8, 2, 128, True)])
def test_qk_norm_rope_kv_many_tokens(nq, nkv, d, gains, per_slot):
    """The 16-bit forms that take a whole token at a time: a block a token (300 tokens), and
    blocks that walk the tokens with the next rows on their way into shared memory (750 tokens);
    more heads than one pass holds, q and k heads sharing a warp, finished rows in between, with and
    without gains."""
    k = K()
    dtype = torch.bfloat16
    eps, theta, n_slots = 1e-6, 10000.0, 3
    t = n_slots * per_slot
    pages = Pages(n_slots, per_slot + 30, nkv, d, dtype, seed=d + nq)
    before_k, before_v = pages.k.clone(), pages.v.clone()
    g = torch.Generator().manual_seed(5)
    slot_of = torch.arange(t) // per_slot
    pos_of = (torch.arange(t) % per_slot) + torch.tensor([0, 30, 7])[slot_of]
    dead = torch.rand(t, generator=g) < 0.1
    pos_of = torch.where(dead, torch.full_like(pos_of, -1), pos_of)
    width = (nq + 2 * nkv) * d
    buf = rnd(t, width + 8, dtype=dtype, seed=11)
    qkv = buf[:, :width]                                  # rows with a stride that is not the width
    orig = qkv.clone()
    qg = 1 + 0.1 * rnd(d, seed=8) if gains else None
    kg = 1 + 0.1 * rnd(d, seed=9) if gains else None
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    freqs = torch.outer(torch.arange(per_slot + 30, dtype=torch.float32), inv)
    positions = pos_of.to(torch.int32).to(DEV)
    slots = slot_of.to(torch.int32).to(DEV)
    k.qk_norm_rope_kv(qkv, t, qg, kg, freqs.cos().to(DEV), freqs.sin().to(DEV), d, positions, slots,
                      pages.k, pages.v, pages.table, nq, nkv, d, eps)

    live = ~dead
    x = orig.cpu().double().view(t, nq + 2 * nkv, d)
    c = freqs[pos_of.clamp(min=0)].double().cos()[:, None, :]
    s_ = freqs[pos_of.clamp(min=0)].double().sin()[:, None, :]

    def rotate(heads, gain):
        if gain is not None:
            heads = heads * torch.rsqrt(heads.pow(2).mean(-1, keepdim=True) + eps) * gain.cpu().double()
        lo, hi = heads[..., : d // 2], heads[..., d // 2:]
        return torch.cat([lo * c - hi * s_, hi * c + lo * s_], -1)

    want_q = rotate(x[:, :nq], qg)
    want_k = rotate(x[:, nq:nq + nkv], kg)
    got_q = qkv.cpu().view(t, nq + 2 * nkv, d)[:, :nq]
    assert rel(got_q[live], want_q[live]) <= TOL[dtype]
    assert torch.equal(qkv[dead.to(DEV)], orig[dead.to(DEV)])
    assert torch.equal(qkv[:, nq * d:], orig[:, nq * d:])             # k and v parts of the rows stay
    table = pages.table.cpu()
    page = table[slot_of, pos_of.clamp(min=0) // 64].long()
    off = pos_of.clamp(min=0) % 64
    got_k, got_v = pages.k.cpu()[page, :, off], pages.v.cpu()[page, :, off]          # [t, nkv, d]
    assert rel(got_k[live], want_k[live]) <= TOL[dtype]
    assert torch.equal(got_v[live], orig.cpu().view(t, -1, d)[:, nq + nkv:][live])
    mask = torch.ones(pages.k.shape[:3], dtype=torch.bool)
    mask[page[live], :, off[live]] = False
    assert torch.equal(pages.k.cpu()[mask], before_k.cpu()[mask])
    assert torch.equal(pages.v.cpu()[mask], before_v.cpu()[mask])
    # the per-head form gives the same rows (a narrow batch takes it)
    q2 = orig[:100].clone()
    k2, v2 = before_k.clone(), before_v.clone()
    k.qk_norm_rope_kv(q2, 100, qg, kg, freqs.cos().to(DEV), freqs.sin().to(DEV), d, positions[:100],
                      slots[:100], k2, v2, pages.table, nq, nkv, d, eps)
    assert rel(q2[:, :nq * d].float(), qkv[:100, :nq * d].float()) <= 1e-2


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (6, 3, 48), (8, 2, 128), (5, 5, 80), (16, 1, 256)])
def test_attention_generic_positions_splits_window(dtype, nq, nkv, d):
    k = K()
    lens = [1, 64, 65, 517, 130]
    pages = Pages(len(lens), max(lens), nkv, d, dtype, seed=3)
    kv = []
    for s, n in enumerate(lens):
        keys, vals = rnd(n, nkv, d, dtype=dtype, seed=10 + s), rnd(n, nkv, d, dtype=dtype, seed=20 + s)
        pages.fill(s, keys, vals)
        kv.append((keys, vals))
    toks = [(0, 0), (1, 63), (2, 64), (3, 516), (3, 0), (3, 255), (4, 129), (4, 64), (2, -1)]
    t = len(toks)
    q = rnd(t, nq * d + 5 * d, dtype=dtype, seed=30)           # rows wider than the q part
    # make one far key stand out for the long sequence: a fault in paging or in the split
    # merge that loses key 3 of 517 changes the result completely
    keys3 = kv[3][0]
    q[3, :d] = (keys3[3, 0].float() * 4).to(dtype)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    for window, splits, per in ((None, 1, 0), (None, 5, 128), (100, 1, 0), (64, 3, 192), (1, 1, 0)):
        out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
        acc = torch.empty(t * nq * max(splits, 1) * d, device=DEV)
        ml = torch.empty(t * nq * max(splits, 1) * 2, device=DEV)
        k.attention_generic(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv, d,
                            scale, window, splits, per, acc, ml)
        for i, (s, p) in enumerate(toks):
            if p < 0:
                assert out[i].abs().max().item() == 0
                continue
            want = ref_attention(q[i, :nq * d].view(nq, d).cpu(), kv[s][0].cpu(), kv[s][1].cpu(), p,
                                 scale, window)
            assert rel(out[i], want) <= TOL[dtype], (window, splits, i)


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 32), (6, 3, 64), (32, 8, 128), (5, 5, 96), (16, 1, 256),
                                      (20, 1, 64), (40, 2, 128)])
def test_attention_decode_bf16(nq, nkv, d):
    """The register-streaming decode kernel: groups of 1 to 20 heads (more than 16 take two
    row blocks), every head size it takes, windows, key splits, finished rows."""
    k = K()
    dtype = torch.bfloat16
    lens = [1, 64, 65, 517, 130, 16, 17]
    pages = Pages(len(lens), max(lens), nkv, d, dtype, seed=5)
    kv = []
    for s, n in enumerate(lens):
        keys, vals = rnd(n, nkv, d, dtype=dtype, seed=10 + s), rnd(n, nkv, d, dtype=dtype, seed=20 + s)
        pages.fill(s, keys, vals)
        kv.append((keys, vals))
    toks = [(0, 0), (1, 63), (2, 64), (3, 516), (3, 0), (3, 255), (4, 129), (4, 64), (2, -1),
            (5, 15), (6, 16), (3, 300)]
    t = len(toks)
    q = rnd(t, nq * d + 2 * nkv * d, dtype=dtype, seed=30)
    q[3, :d] = (kv[3][0][3, 0].float() * 4).to(dtype)          # one far key dominates
    q[11, (nq - 1) * d:nq * d] = (kv[3][0][299, nkv - 1].float() * 4).to(dtype)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    for window, splits, per in ((None, 1, 0), (None, 5, 128), (None, 9, 64), (100, 1, 0), (64, 3, 192),
                                (1, 1, 0), (17, 33, 16), (None, 6, 0), (100, 4, 0), (None, 48, 0)):
        out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
        acc = torch.empty(t * nq * max(splits, 1) * d, device=DEV)
        ml = torch.empty(t * nq * max(splits, 1) * 2, device=DEV)
        k.attention_decode_bf16(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv,
                                d, scale, window, splits, per, acc, ml)
        for i, (s, p) in enumerate(toks):
            if p < 0:
                assert out[i].abs().max().item() == 0
                continue
            want = ref_attention(q[i, :nq * d].view(nq, d).cpu(), kv[s][0].cpu(), kv[s][1].cpu(), p,
                                 scale, window)
            assert rel(out[i], want) <= TOL[dtype], (window, splits, i)


@pytest.mark.parametrize("nq,nkv,d", [(6, 3, 64), (32, 8, 128), (5, 5, 64), (16, 1, 128), (40, 4, 128),
                                      (3, 1, 64)])
def test_attention_decode_tma(nq, nkv, d):
    """The TMA-fed decode kernel: groups of 1 to 16 heads, both head sizes, windows, 1 to 8 splits
    as clusters (more splits than a short sequence has pages), finished rows, one far key."""
    k = K()
    dtype = torch.bfloat16
    lens = [1, 64, 65, 1100, 130, 16, 17]
    pages = Pages(len(lens), max(lens), nkv, d, dtype, seed=5)
    kv = []
    for s, n in enumerate(lens):
        keys, vals = rnd(n, nkv, d, dtype=dtype, seed=10 + s), rnd(n, nkv, d, dtype=dtype, seed=20 + s)
        pages.fill(s, keys, vals)
        kv.append((keys, vals))
    toks = [(0, 0), (1, 63), (2, 64), (3, 1099), (3, 0), (3, 255), (4, 129), (4, 64), (2, -1),
            (5, 15), (6, 16), (3, 300), (3, 1023), (3, 1024)]
    t = len(toks)
    q = rnd(t, nq * d + 2 * nkv * d, dtype=dtype, seed=30)
    q[3, :d] = (kv[3][0][3, 0].float() * 4).to(dtype)          # one far key dominates
    q[11, (nq - 1) * d:nq * d] = (kv[3][0][299, nkv - 1].float() * 4).to(dtype)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    cases = [(None, 1), (None, 2), (None, 5), (None, 8), (100, 1), (64, 3), (1, 1), (17, 8), (700, 4)]
    most = k.decode_tma_max_splits(d, DEV)
    if most > 8:                                   # clusters of more than the portable 8 blocks
        cases += [(None, 16), (None, 11), (300, 13)]
    for window, splits in cases:
        out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
        k.attention_decode_tma(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv, d,
                               scale, window, splits)
        k.check_tc_status(DEV)
        for i, (s, p) in enumerate(toks):
            if p < 0:
                assert out[i].abs().max().item() == 0
                continue
            want = ref_attention(q[i, :nq * d].view(nq, d).cpu(), kv[s][0].cpu(), kv[s][1].cpu(), p,
                                 scale, window)
            assert rel(out[i], want) <= TOL[dtype], (window, splits, i)
    # it refuses what it cannot take
    from enginekernel_b200.ops.lib import KernelError
    with pytest.raises(KernelError):
        k.attention_decode_tma(out, q, t, positions, slots, pages.k, pages.v, pages.table, nq, nkv, d,
                               scale, None, most + 1)


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (6, 2, 48), (32, 8, 128), (5, 5, 80), (16, 1, 256),
                                      (3, 1, 64), (8, 2, 128), (16, 2, 64), (4, 4, 128), (64, 1, 64)])
def test_attention_prefill_bf16(nq, nkv, d):
    """The prompt kernel: several sequences of unequal lengths in one launch, some of them
    continuing after tokens already in the cache, groups that do not divide 128, windows."""
    k = K()
    dtype = torch.bfloat16
    # (length of the sequence, first new token)
    seqs = [(1, 0), (64, 0), (65, 0), (517, 0), (130, 100), (200, 199), (300, 37)]
    pages = Pages(len(seqs), max(n for n, _ in seqs), nkv, d, dtype, seed=7)
    kv, rows, positions, slots, cu = [], [], [], [], [0]
    for s, (n, start) in enumerate(seqs):
        keys, vals = rnd(n, nkv, d, dtype=dtype, seed=10 + s), rnd(n, nkv, d, dtype=dtype, seed=20 + s)
        pages.fill(s, keys, vals)
        kv.append((keys, vals))
        for p in range(start, n):
            rows.append((s, p))
            positions.append(p)
            slots.append(s)
        cu.append(len(rows))
    t = len(rows)
    q = rnd(t, nq * d + 2 * nkv * d, dtype=dtype, seed=30)
    far = rows.index((3, 516))
    q[far, :d] = (kv[3][0][3, 0].float() * 4).to(dtype)            # one far key dominates
    positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    variants = [k.attention_prefill_bf16]
    if k.attention_prefill_tc_supported(dtype, d, nq, nkv):
        variants.append(k.attention_prefill_tc)          # the tcgen05 kernel, same contract
    for window, fn in [(w, f) for f in variants for w in (None, 100, 1, 64)]:
        out = torch.full((t, nq * d), 7.0, dtype=dtype, device=DEV)
        fn(out, q, t, positions, slots, cu_t, len(seqs), pages.k, pages.v, pages.table, nq, nkv, d,
           scale, window)
        if fn is k.attention_prefill_tc:
            k.check_tc_status(DEV)
        outc, qc = out.cpu(), q.cpu()
        worst = 0.0
        for i in range(0, t, 7 if t > 200 else 1):
            s, p = rows[i]
            want = ref_attention(qc[i, :nq * d].view(nq, d), kv[s][0].cpu(), kv[s][1].cpu(), p, scale, window)
            worst = max(worst, rel(outc[i], want))
        for i in (far, t - 1, cu[4], cu[5], cu[6]):
            s, p = rows[i]
            want = ref_attention(qc[i, :nq * d].view(nq, d), kv[s][0].cpu(), kv[s][1].cpu(), p, scale, window)
            worst = max(worst, rel(outc[i], want))
        assert worst <= TOL[dtype], (window, fn.__name__, worst)


# ------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("m,n,k_", [(1, 331, 80), (3, 2560, 176), (16, 100, 33), (17, 65, 64),
                                    (130, 384, 96), (64, 1, 1)])
def test_gemm_f32_is_true_32_bit(m, n, k_):
    k = K()
    x, w = rnd(m, k_, seed=1), rnd(n, k_, seed=2)
    out = torch.empty(m, n, device=DEV)
    k.gemm_f32(out, x, w)
    want = x.double() @ w.double().t()
    assert rel(out, want) <= 2e-6
    # a TF32 product would be off by ~1e-3 here
    # rows do not depend on their batch mates, bit for bit
    if m > 1:
        one = torch.empty(1, n, device=DEV)
        k.gemm_f32(one, x[m - 1:m].contiguous(), w)
        assert torch.equal(one[0], out[m - 1])


@pytest.mark.parametrize("m,n,k_", [(17, 256, 128), (64, 2560, 4096), (33, 1000, 1000), (1, 128, 64),
                                    (48, 331 * 2, 80), (64, 6144, 2560), (24, 1280, 2560),
                                    (24, 20012, 2560)])
def test_gemm_tc_swapped(m, n, k_):
    """tcgen05 + TMA product with the weights on the 128-row side (decode with many sequences)."""
    k = K()
    x = rnd(m, k_, dtype=torch.bfloat16, seed=1)
    w = rnd(n, k_, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.double() @ w.double().t()
    # K split over the blocks of a cluster (up to 8), through scratch in global memory (forced, or
    # more than 8 splits), or not at all
    for k_split, cluster in ((1, True), (3, True), (3, False), (8, True), (11, True), (None, True)):
        out32 = torch.full((m, n), 9.0, device=DEV)
        k.gemm_tc_bf16(out32, x, w, k.EPI_F32, swap=True, k_split=k_split, cluster=cluster)
        k.check_tc_status(DEV)
        assert rel(out32, want) <= 1e-5, (k_split, cluster)
        out16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        k.gemm_tc_bf16(out16, x, w, k.EPI_BF16, swap=True, k_split=k_split, cluster=cluster)
        assert rel(out16, want) <= 4e-3
        inter = n // 2
        act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
        k.gemm_tc_bf16(act, x, w, k.EPI_SWIGLU, swap=True, k_split=k_split, cluster=cluster)
        g, u = want[:, :inter], want[:, inter:]
        assert rel(act, g / (1 + torch.exp(-g)) * u) <= 4e-3, (k_split, cluster)
    # the same split gives the same bits whichever way the partial tiles are added
    a32, b32 = torch.empty(m, n, device=DEV), torch.empty(m, n, device=DEV)
    k.gemm_tc_bf16(a32, x, w, k.EPI_F32, swap=True, k_split=3, cluster=True)
    k.gemm_tc_bf16(b32, x, w, k.EPI_F32, swap=True, k_split=3, cluster=False)
    assert torch.equal(a32, b32)
    k.check_tc_status(DEV)
    _, tickets = k.split_scratch(DEV)
    assert int(tickets.abs().sum()) == 0


@pytest.mark.parametrize("m,n,k_", [(8, 2560, 4096), (1, 256, 128), (33, 1000, 1000), (64, 1024, 3072),
                                    (5, 136, 80)])
def test_gemm_tc_deferred_norm(m, n, k_):
    """The two halves of a norm moved into the products around it: the product before adds its
    result to the stream, leaves stream * gain and the tiles' sums of squares; the product after
    scales its rows by the 1/rms those sums give (also under SwiGLU)."""
    k = K()
    x = rnd(m, k_, dtype=torch.bfloat16, seed=1)
    w = rnd(n, k_, dtype=torch.bfloat16, seed=2, scale=0.05)
    stream0 = rnd(m + 2, n, seed=3, scale=2.0)
    gain = 1 + 0.1 * rnd(n, seed=4)
    eps = 1e-5
    tiles = -(-n // 128)
    for k_split in (None, 1, 3):
        stream = stream0.clone()
        scaled = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
        ss = torch.full((m, tiles), -1.0, device=DEV)
        k.gemm_tc_bf16(scaled, x, w, k.EPI_BF16, swap=True, k_split=k_split, residual=(stream, gain, ss))
        k.check_tc_status(DEV)
        want_stream = stream0[:m].double() + x.double() @ w.double().t()
        assert rel(stream[:m], want_stream) <= 1e-5
        assert torch.equal(stream[m:], stream0[m:])                   # rows beyond m are not touched
        assert rel(scaled, want_stream * gain.double()) <= 4e-3
        assert rel(ss.sum(1), want_stream.pow(2).sum(1)) <= 1e-5
        pad = torch.nn.functional.pad(stream[:m].double().pow(2), (0, tiles * 128 - n))
        assert rel(ss, pad.view(m, tiles, 128).sum(-1)) <= 1e-5
        # the consumer: y = rmsnorm(stream) * gain, then y . w2^T, from `scaled` and `ss`
        n2 = 384
        w2 = rnd(n2, n, dtype=torch.bfloat16, seed=5, scale=0.05)
        rstd = torch.rsqrt(stream[:m].double().pow(2).mean(1, keepdim=True) + eps)
        want = (scaled.double() * rstd) @ w2.double().t()
        out = torch.empty(m, n2, dtype=torch.bfloat16, device=DEV)
        k.gemm_tc_bf16(out, scaled, w2, k.EPI_BF16, swap=True, k_split=k_split, row_scale=(ss, n, eps))
        assert rel(out, want) <= 4e-3
        out32 = torch.empty(m, n2, device=DEV)
        k.gemm_tc_bf16(out32, scaled, w2, k.EPI_F32, swap=True, k_split=k_split, row_scale=(ss, n, eps))
        assert rel(out32, want) <= 1e-5
        act = torch.empty(m, n2 // 2, dtype=torch.bfloat16, device=DEV)
        k.gemm_tc_bf16(act, scaled, w2, k.EPI_SWIGLU, swap=True, k_split=k_split, row_scale=(ss, n, eps))
        g, u = want[:, :n2 // 2], want[:, n2 // 2:]
        assert rel(act, g / (1 + torch.exp(-g)) * u) <= 4e-3
    k.check_tc_status(DEV)


@pytest.mark.parametrize("m,nq,nkv,hidden,gains", [(8, 32, 8, 2560, True), (1, 4, 2, 256, True),
                                                    (37, 6, 3, 200, False), (64, 16, 8, 1024, True),
                                                    (24, 8, 2, 2560, True)])
def test_gemm_tc_qkv_rope(m, nq, nkv, hidden, gains):
    """The q/k/v product with head norm, rotation and cache write in its epilogue, against the
    product followed by qk_norm_rope_kv: finished rows, pages in shuffled order, no cache write,
    a row scale from a deferred norm."""
    k = K()
    d, dtype = 128, torch.bfloat16
    eps, theta, n_slots, max_len = 1e-6, 10000.0, 5, 300
    n = (nq + 2 * nkv) * d
    x = rnd(m, hidden, dtype=dtype, seed=1)
    w = rnd(n, hidden, dtype=dtype, seed=2, scale=0.05)
    qg = 1 + 0.1 * rnd(d, seed=8) if gains else None
    kg = 1 + 0.1 * rnd(d, seed=9) if gains else None
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    freqs = torch.outer(torch.arange(max_len, dtype=torch.float32), inv)
    cos, sin = freqs.cos().to(DEV), freqs.sin().to(DEV)
    g = torch.Generator().manual_seed(m)
    slot_of = torch.randint(0, n_slots, (m,), generator=g)
    pos_of = torch.randint(0, max_len, (m,), generator=g)
    pos_of[torch.rand(m, generator=g) < 0.15] = -1
    # two tokens must not share a cache place
    seen = set()
    for i in range(m):
        while pos_of[i] >= 0 and (int(slot_of[i]), int(pos_of[i])) in seen:
            pos_of[i] = (pos_of[i] + 1) % max_len
        seen.add((int(slot_of[i]), int(pos_of[i])))
    positions, slots = pos_of.to(torch.int32).to(DEV), slot_of.to(torch.int32).to(DEV)
    ss = (rnd(m, 3, seed=4).abs() + 0.5) * hidden / 3
    for write_kv, row_scale in ((True, None), (False, None), (True, (ss, hidden, 1e-5))):
        # the two-kernel way
        pa = Pages(n_slots, max_len, nkv, d, dtype, seed=3)
        ref = torch.empty(m, n, dtype=dtype, device=DEV)
        k.gemm_tc_bf16(ref, x, w, k.EPI_BF16, swap=True, row_scale=row_scale)
        k.qk_norm_rope_kv(ref, m, qg, kg, cos, sin, d, positions, slots, pa.k, pa.v, pa.table, nq, nkv, d,
                          eps, write_kv=write_kv)
        # the fused way
        pb = Pages(n_slots, max_len, nkv, d, dtype, seed=3)
        got = torch.full((m, n), 7.0, dtype=dtype, device=DEV)
        k.gemm_tc_qkv_rope(got, x, w, m, qg, kg, eps, cos, sin, positions, slots, pb.k, pb.v, pb.table,
                           nq, nkv, write_kv=write_kv, row_scale=row_scale)
        k.check_tc_status(DEV)
        live = (pos_of >= 0).to(DEV)
        # q: one rounding instead of two, so equal up to a bfloat16 ulp of the largest value
        assert rel(got[live][:, :nq * d], ref[live][:, :nq * d]) <= 1e-2, (write_kv, row_scale is not None)
        assert rel(pb.k, pa.k) <= 1e-2 and rel(pb.v, pa.v) <= 1e-2
        assert torch.equal(pb.v, pa.v)                        # values are copied, not computed
        if not write_kv:
            assert pb.k.abs().sum().item() == 0 and pb.v.abs().sum().item() == 0
    # against 64-bit arithmetic, for one live row
    i = int(torch.nonzero(pos_of >= 0)[0])
    full = (x[i].double() @ w.double().t()).view(nq + 2 * nkv, d).cpu()
    c, s_ = freqs[pos_of[i]].double().cos(), freqs[pos_of[i]].double().sin()

    def rot(h, gain):
        if gain is not None:
            h = h * torch.rsqrt(h.pow(2).mean() + eps) * gain.double().cpu()
        lo, hi = h[: d // 2], h[d // 2:]
        return torch.cat([lo * c - hi * s_, hi * c + lo * s_])
    pb = Pages(n_slots, max_len, nkv, d, dtype, seed=3)
    got = torch.empty(m, n, dtype=dtype, device=DEV)
    k.gemm_tc_qkv_rope(got, x, w, m, qg, kg, eps, cos, sin, positions, slots, pb.k, pb.v, pb.table, nq, nkv)
    for h in range(nq):
        assert rel(got[i, h * d:(h + 1) * d], rot(full[h], qg)) <= TOL[dtype]
    page = int(pb.table[slot_of[i], pos_of[i] // 64])
    for h in range(nkv):
        assert rel(pb.k[page, h, pos_of[i] % 64], rot(full[nq + h], kg)) <= TOL[dtype]
        assert rel(pb.v[page, h, pos_of[i] % 64], full[nq + nkv + h]) <= TOL[dtype]


@pytest.mark.parametrize("m,n,k_", [(128, 128, 64), (2048, 2560, 4096), (300, 1000, 1000), (65, 662, 80),
                                    (517, 6144, 2560)])
def test_gemm_tc_direct(m, n, k_):
    """tcgen05 + TMA product in 128 x 128 output tiles (prompts), edges not multiples of a tile."""
    k = K()
    x = rnd(m, k_, dtype=torch.bfloat16, seed=3)
    w = rnd(n, k_, dtype=torch.bfloat16, seed=4, scale=0.05)
    want = x.double() @ w.double().t()
    out32 = torch.full((m, n), 9.0, device=DEV)
    k.gemm_tc_bf16(out32, x, w, k.EPI_F32, swap=False)
    k.check_tc_status(DEV)
    assert rel(out32, want) <= 1e-5
    out16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    k.gemm_tc_bf16(out16, x, w, k.EPI_BF16, swap=False)
    assert rel(out16, want) <= 4e-3
    inter = n // 2
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    k.gemm_tc_bf16(act, x, w, k.EPI_SWIGLU, swap=False)
    g, u = want[:, :inter], want[:, inter:]
    assert rel(act, g / (1 + torch.exp(-g)) * u) <= 4e-3
    k.check_tc_status(DEV)


@pytest.mark.parametrize("lengths,starts,group,d", [((5, 300, 64, 129), (0, 0, 0, 0), 4, 128),
                                                     ((40, 33), (1000, 10), 2, 64),
                                                     ((1,) * 37, (0,) * 37, 8, 128), ((700,), (0,), 1, 64),
                                                     ((9000, 3000, 8000, 70, 12000), (0, 4000, 100, 0, 0), 4, 128)])
def test_prefill_tile_table(lengths, starts, group, d):
    """The table of tiles of the tcgen05 prompt attention: every token in exactly one tile, a tile
    within one sequence; the sequences by the length of their context in bands that fit L2, the bands
    one after another, inside a band the last tiles of its sequences first; empty entries behind."""
    k = K()
    n_q, n_kv = 8 * group, 8
    per = k.PREFILL_TC_ROWS // group
    cu = [0]
    pos, slot = [], []
    for b, (n, a) in enumerate(zip(lengths, starts)):
        cu.append(cu[-1] + n)
        pos += list(range(a, a + n))
        slot += [10 + b] * n
    n_tokens = cu[-1]
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tiles = torch.full((-(-n_tokens // per) + len(lengths) + 5, 4), -7, dtype=torch.int32, device=DEV)
    n = k.attention_prefill_tiles(tiles, n_tokens, as_dev(pos), as_dev(slot), as_dev(cu), len(lengths), n_q, n_kv, d)
    got = tiles[:n].cpu().tolist()
    assert bool((tiles[n:] == -7).all())                    # nothing written past what was asked for
    live = [e for e in got if e[1] > 0]
    assert all(e[1] == 0 for e in got[len(live):])          # the empty entries stand behind
    covered = sorted(t for first, count, _, _ in live for t in range(first, first + count))
    assert covered == list(range(n_tokens))
    budget = k.prefill_band_tokens(n_kv, d, DEV)
    order = sorted(range(len(lengths)), key=lambda b: (-(starts[b] + lengths[b]), b))
    bands, held = [[]], 0
    for b in order:
        if bands[-1] and held + starts[b] + lengths[b] > budget:
            bands.append([])
            held = 0
        bands[-1].append(b)
        held += starts[b] + lengths[b]
    if len(lengths) == 5:
        assert len(bands) > 1                               # (the long case does not fit one band)
    want = []
    for band in bands:
        most = max(-(-lengths[b] // per) for b in band)
        for r in reversed(range(most)):
            for b in band:
                if r < -(-lengths[b] // per):
                    want.append([cu[b] + r * per, min(per, lengths[b] - r * per), starts[b] + r * per, 10 + b])
    assert live == want


@pytest.mark.parametrize("m,n,k_", [(256, 256, 64), (300, 528, 200), (65, 1040, 72), (1000, 6144, 2560),
                                    (2048, 2560, 4096), (5000, 784, 320)])
def test_gemm_pair(m, n, k_):
    """The product on pairs of SMs (tcgen05.mma.cta_group::2, 256 x 256 tiles, persistent), its three
    epilogues, with edges that are no multiples of a tile and more tiles than pairs."""
    k = K()
    x = rnd(m, k_, dtype=torch.bfloat16, seed=3)
    w = rnd(n, k_, dtype=torch.bfloat16, seed=4, scale=0.05)
    want = x.double() @ w.double().t()
    out16 = torch.full((m + 3, n), 9.0, dtype=torch.bfloat16, device=DEV)
    k.gemm_pair_bf16(out16, x, w, k.PAIR_EPI_BF16, n_rows=m)
    k.check_tc_status(DEV)
    assert rel(out16[:m], want) <= 4e-3
    assert bool((out16[m:] == 9.0).all())                 # rows beyond the product stay as they were
    base = rnd(m, n, seed=5)
    stream = base.clone()
    k.gemm_pair_bf16(stream, x, w, k.PAIR_EPI_ADD_F32)
    assert rel(stream, base.double() + want) <= 1e-5
    inter = n // 2
    act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    k.gemm_pair_bf16(act, x, w, k.PAIR_EPI_SWIGLU)
    g, u = want[:, :inter], want[:, inter:]
    assert rel(act, g / (1 + torch.exp(-g)) * u) <= 4e-3
    k.check_tc_status(DEV)


@pytest.mark.parametrize("m,nq,nkv,hidden,gains", [(300, 4, 2, 320, True), (1000, 3, 1, 136, True),
                                                   (777, 8, 8, 512, False)])
def test_gemm_pair_qkv_rope(m, nq, nkv, hidden, gains):
    """The q/k/v product of many rows with head norm, rotation and cache write in its epilogue,
    against the same product followed by the rotation kernel, and against 64-bit arithmetic; an
    odd number of heads leaves the last tile half empty."""
    k = K()
    d, dtype = 128, torch.bfloat16
    eps, theta, n_slots, max_len = 1e-6, 10000.0, 7, 400
    n = (nq + 2 * nkv) * d
    x = rnd(m, hidden, dtype=dtype, seed=1)
    w = rnd(n, hidden, dtype=dtype, seed=2, scale=0.05)
    qg = 1 + 0.1 * rnd(d, seed=8) if gains else None
    kg = 1 + 0.1 * rnd(d, seed=9) if gains else None
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    freqs = torch.outer(torch.arange(max_len, dtype=torch.float32), inv)
    cos, sin = freqs.cos().to(DEV), freqs.sin().to(DEV)
    g = torch.Generator().manual_seed(m)
    # every token its own cache place; some rows are dead
    place = torch.randperm(n_slots * max_len, generator=g)[:m]
    slot_of, pos_of = place // max_len, place % max_len
    pos_of[torch.rand(m, generator=g) < 0.1] = -1
    positions, slots = pos_of.to(torch.int32).to(DEV), slot_of.to(torch.int32).to(DEV)
    live = (pos_of >= 0).to(DEV)
    for write_kv in (True, False):
        pa = Pages(n_slots, max_len, nkv, d, dtype, seed=3)
        ref = torch.empty(m, n, dtype=dtype, device=DEV)
        k.gemm_pair_bf16(ref, x, w, k.PAIR_EPI_BF16)
        k.qk_norm_rope_kv(ref, m, qg, kg, cos, sin, d, positions, slots, pa.k, pa.v, pa.table, nq, nkv, d,
                          eps, write_kv=write_kv)
        pb = Pages(n_slots, max_len, nkv, d, dtype, seed=3)
        got = torch.full((m, n), 7.0, dtype=dtype, device=DEV)
        k.gemm_pair_qkv_rope(got, x, w, m, qg, kg, eps, cos, sin, positions, slots, pb.k, pb.v, pb.table,
                             nq, nkv, write_kv=write_kv)
        k.check_tc_status(DEV)
        # one rounding instead of two: equal up to a bfloat16 ulp of the largest value
        assert rel(got[live][:, :nq * d], ref[live][:, :nq * d]) <= 1e-2, write_kv
        assert bool((got[~live] == 7.0).all())                # dead rows are not touched
        assert rel(pb.k, pa.k) <= 1e-2
        assert torch.equal(pb.v, pa.v)                        # values: the same sums, rounded once
        if not write_kv:
            assert pb.k.abs().sum().item() == 0 and pb.v.abs().sum().item() == 0
    i = int(torch.nonzero(pos_of >= 0)[-1])
    full = (x[i].double() @ w.double().t()).view(nq + 2 * nkv, d).cpu()
    c, s_ = freqs[pos_of[i]].double().cos(), freqs[pos_of[i]].double().sin()

    def rot(h, gain):
        if gain is not None:
            h = h * torch.rsqrt(h.pow(2).mean() + eps) * gain.double().cpu()
        lo, hi = h[: d // 2], h[d // 2:]
        return torch.cat([lo * c - hi * s_, hi * c + lo * s_])
    pb = Pages(n_slots, max_len, nkv, d, dtype, seed=3)
    got = torch.empty(m, n, dtype=dtype, device=DEV)
    k.gemm_pair_qkv_rope(got, x, w, m, qg, kg, eps, cos, sin, positions, slots, pb.k, pb.v, pb.table, nq, nkv)
    for h in range(nq):
        assert rel(got[i, h * d:(h + 1) * d], rot(full[h], qg)) <= TOL[dtype]
    page = int(pb.table[slot_of[i], pos_of[i] // 64])
    for h in range(nkv):
        assert rel(pb.k[page, h, pos_of[i] % 64], rot(full[nq + h], kg)) <= TOL[dtype]
        assert rel(pb.v[page, h, pos_of[i] % 64], full[nq + nkv + h]) <= TOL[dtype]


def test_gemm_pair_refuses_rows_it_cannot_address():
    k = K()
    from enginekernel_b200.ops.lib import KernelError
    x = rnd(300, 64, dtype=torch.bfloat16)
    w = rnd(520, 64, dtype=torch.bfloat16)
    with pytest.raises(KernelError):                      # 260 outputs a row: rows not 16-byte aligned
        k.gemm_pair_bf16(torch.empty(300, 260, dtype=torch.bfloat16, device=DEV), x, w, k.PAIR_EPI_SWIGLU)
    with pytest.raises(KernelError):                      # the add form wants the 32-bit stream
        k.gemm_pair_bf16(torch.empty(300, 520, dtype=torch.bfloat16, device=DEV), x, w, k.PAIR_EPI_ADD_F32)


def test_launchers_refuse_what_they_cannot_do():
    k = K()
    from enginekernel_b200.ops.lib import KernelError
    x = rnd(2, 12, dtype=torch.bfloat16)
    w = rnd(16, 12, dtype=torch.bfloat16)
    with pytest.raises(KernelError):                      # inner size 12 is no multiple of 8
        k.gemm_tc_bf16(torch.empty(2, 16, dtype=torch.bfloat16, device=DEV), x, w)
    with pytest.raises(KernelError):
        k.check_head_dim(24)
    with pytest.raises(KernelError):
        k.rmsnorm(torch.empty(1, 8), torch.empty(1, 8), torch.empty(8), 1e-6)   # CPU tensors


# ------------------------------------------------------------------ sampling and state
def test_sample_greedy_gumbel_topk():
    k = K()
    vocab = 1000
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(5, vocab, generator=g) * 3).to(DEV)
    logits[1, 17] = logits[1, 900] = 50.0                 # a tie: the lower index wins
    out = torch.full((5,), -5, dtype=torch.int32, device=DEV)
    k.sample(out, logits, 0.0, 0, 0)
    assert out.tolist() == [int(torch.argmax(r)) for r in logits.cpu()] and out[1].item() == 17

    streams = torch.tensor([4, 0, 9, 2, 2], dtype=torch.int32, device=DEV)
    draws = torch.tensor([0, 3, 1, 7, 8], dtype=torch.int32, device=DEV)
    active = torch.tensor([5, 5, -1, 5, 5], dtype=torch.int32, device=DEV)
    for temp, topk, seed in ((0.8, 0, 1234), (1.5, 3, 7), (0.3, 50, (1 << 40) + 5)):
        out.fill_(-5)
        k.sample(out, logits, temp, topk, seed, streams=streams, draws=draws, active=active)
        dyn = torch.full((5,), -5, dtype=torch.int32, device=DEV)
        k.sample(dyn, logits, 0.0, 0, 0, streams=streams, draws=draws, active=active,
                 dyn=k.sampling_settings(temp, topk, seed, DEV))
        assert torch.equal(out, dyn)
        for r in range(5):
            if r == 2:
                assert out[r].item() == -5                # inactive rows are left alone
                continue
            want = plain.sample_token(logits[r].cpu(), temp, topk, seed, int(streams[r]), int(draws[r]))
            assert out[r].item() == want, (temp, topk, r)


def test_sample_wide_equals_the_one_block_kernel():
    k = K()
    for vocab in (4099, 151936):
        g = torch.Generator().manual_seed(vocab)
        logits = (torch.randn(6, vocab, generator=g) * 2).to(DEV)
        logits[2, 5] = logits[2, vocab - 1] = 40.0            # a tie across segments
        streams = torch.tensor([3, 1, 4, 1, 5, 9], dtype=torch.int32, device=DEV)
        draws = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32, device=DEV)
        active = torch.tensor([1, 1, 1, -1, 1, 1], dtype=torch.int32, device=DEV)
        ps = torch.empty(6 * k.SAMPLE_SEGMENTS, device=DEV)
        pi = torch.empty(6 * k.SAMPLE_SEGMENTS, dtype=torch.int32, device=DEV)
        for temp, seed in ((0.0, 0), (0.9, 77), (2.0, (1 << 35) + 1)):
            one = torch.full((6,), -5, dtype=torch.int32, device=DEV)
            wide = torch.full((6,), -5, dtype=torch.int32, device=DEV)
            k.sample(one, logits, temp, 0, seed, streams=streams, draws=draws, active=active)
            k.sample_wide(wide, logits, temp, seed, ps, pi, streams=streams, draws=draws, active=active)
            assert torch.equal(one, wide) and wide[3].item() == -5
            dyn = torch.full((6,), -5, dtype=torch.int32, device=DEV)
            k.sample_wide(dyn, logits, 0.0, 0, ps, pi, streams=streams, draws=draws, active=active,
                          dyn=k.sampling_settings(temp, 0, seed, DEV))
            assert torch.equal(dyn, wide)
        if temp == 0.0:
            assert wide[2].item() == 5


def test_sample_cluster_equals_the_one_block_kernel():
    """Eight blocks a row as a cluster: the same token as the one-block kernel in every mode, with
    ties at the top-k threshold, ties across pieces, top_k of 1 and of nearly the vocabulary, NaN
    and -inf entries, rows switched off, settings read from the device."""
    k = K()
    for vocab in (4099, 151936, 50):
        g = torch.Generator().manual_seed(vocab)
        logits = (torch.randn(6, vocab, generator=g) * 2).to(DEV)
        logits[2, 5] = logits[2, vocab - 1] = 40.0            # a tie across pieces
        logits[4, :40] = 3.25                                  # many equal values around a threshold
        logits[5, 7] = float("nan")
        logits[5, 11] = float("-inf")
        streams = torch.tensor([3, 1, 4, 1, 5, 9], dtype=torch.int32, device=DEV)
        draws = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32, device=DEV)
        active = torch.tensor([1, 1, 1, -1, 1, 1], dtype=torch.int32, device=DEV)
        for temp, topk, seed in ((0.0, 0, 0), (0.9, 0, 77), (0.9, 50, 77), (1.3, 1, 5), (0.7, 17, (1 << 35) + 1),
                                 (1.0, vocab - 1, 9), (1.0, vocab + 5, 9), (2.0, 1000, 3)):
            one = torch.full((6,), -5, dtype=torch.int32, device=DEV)
            many = torch.full((6,), -5, dtype=torch.int32, device=DEV)
            k.sample(one, logits, temp, topk, seed, streams=streams, draws=draws, active=active)
            k.sample_cluster(many, logits, temp, topk, seed, streams=streams, draws=draws, active=active)
            assert torch.equal(one, many) and many[3].item() == -5, (vocab, temp, topk)
            dyn = torch.full((6,), -5, dtype=torch.int32, device=DEV)
            k.sample_cluster(dyn, logits, 0.0, 0, 0, streams=streams, draws=draws, active=active,
                             dyn=k.sampling_settings(temp, topk, seed, DEV))
            assert torch.equal(dyn, many)


def test_sample_distribution():
    """Many draws of one row follow softmax(logits / T)."""
    k = K()
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]], device=DEV).repeat(4000, 1)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    draws = torch.arange(4000, dtype=torch.int32, device=DEV)
    streams = torch.zeros(4000, dtype=torch.int32, device=DEV)
    k.sample(out, logits, 0.7, 0, 99, streams=streams, draws=draws)
    freq = torch.bincount(out.long().cpu(), minlength=5).double() / 4000
    want = torch.softmax(logits[0].double().cpu() / 0.7, -1)
    assert (freq - want).abs().max().item() < 0.03


def test_decode_advance():
    k = K()
    b = 5
    i32 = dict(dtype=torch.int32, device=DEV)
    sampled = torch.tensor([11, 99, 13, 14, 15], **i32)
    tokens = torch.tensor([1, 2, 3, 4, 5], **i32)
    positions = torch.tensor([10, 20, -1, 40, 50], **i32)
    draws = torch.zeros(b, **i32)
    remaining = torch.tensor([5, 5, 5, 1, 5], **i32)
    out = torch.full((4, b), -7, **i32)
    step = torch.tensor([2], **i32)
    stop = torch.tensor([99, 98], **i32)
    k.decode_advance(sampled, tokens, positions, draws, remaining, out, step, stop, 2, b)
    assert out[2].tolist() == [11, 99, -1, 14, 15] and step.item() == 3
    assert positions.tolist() == [11, -1, -1, -1, 51]     # stop token, finished, budget used up
    assert tokens.tolist() == [11, 2, 3, 4, 15]
    assert draws.tolist() == [1, 1, 0, 1, 1] and remaining.tolist() == [4, 4, 5, 0, 4]
    assert (out[[0, 1, 3]] == -7).all()


def test_a_wait_that_runs_out_reaches_the_caller_and_is_cleared():
    """Every barrier wait in the tensor-core kernels gives up after a limit, records a code in the
    device's status word and lets its kernel end.  Here a one-thread kernel waits 4,096 rounds for a
    barrier that nothing completes (it ends by itself, in well under a millisecond): the check
    raises with the code, the word is clear afterwards, and a product right after it is correct."""
    k = K()
    from enginekernel_b200.ops.lib import KernelError
    k.check_tc_status(DEV)                                   # clean before
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    k.wait_that_runs_out(DEV, code=77, limit=4096)
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 100.0                       # milliseconds: the wait was bounded
    with pytest.raises(KernelError, match="code 77"):
        k.check_tc_status(DEV)
    k.check_tc_status(DEV)                                   # cleared by the check that raised
    assert int(k.tc_status(DEV).item()) == 0
    x = rnd(8, 256, dtype=torch.bfloat16, seed=1)
    w = rnd(384, 256, dtype=torch.bfloat16, seed=2, scale=0.05)
    out = torch.empty(8, 384, device=DEV)
    k.gemm_tc_bf16(out, x, w, k.EPI_F32, swap=True)
    assert rel(out, x.double() @ w.double().t()) <= 1e-5
    k.check_tc_status(DEV)
    # the first code wins until the word is read
    k.wait_that_runs_out(DEV, code=5, limit=256)
    k.wait_that_runs_out(DEV, code=6, limit=256)
    with pytest.raises(KernelError, match="code 5"):
        k.check_tc_status(DEV)
    with pytest.raises(KernelError):
        k.wait_that_runs_out(DEV, code=1, limit=10**9)       # refused: only short waits
