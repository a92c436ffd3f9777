"""sm_100a kernels against plain PyTorch fp32 references of the same op (small cases)."""
import math

import numpy as np
import pytest
import torch

from rexl3_b200.format import exl3

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.ops import kernels
    return kernels


def _mk(K, k, n, bits, cb="3inst", seed=0, out_scale=0.05):
    rng = np.random.default_rng(seed)
    b = exl3.Bits.of(bits)
    tr = exl3.random_trellis(k // 16, n // 16, b, seed)
    suh = rng.uniform(0.5, 1.5, k).astype(np.float16) * np.where(rng.random(k) < 0.5, -1, 1).astype(np.float16)
    svh = rng.uniform(0.5, 1.5, n).astype(np.float16) * np.float16(out_scale)
    return K.Exl3Weight.from_numpy(tr, suh, svh, None, cb), tr, suh, svh


def test_unpack_bit_exact_every_width_and_codebook(K):
    for cb in exl3.CODEBOOKS:
        for t in exl3.ALL_TWICE:
            if t % 2 and cb != "mul1":
                continue
            tr = exl3.random_trellis(8, 8, exl3.Bits(t), seed=t)
            w = K.Exl3Weight.from_numpy(tr, np.ones(128, np.float16), np.ones(128, np.float16), None, cb)
            got = K.exl3_unpack(w).cpu().numpy().view(np.uint16)
            assert np.array_equal(got, exl3.unpack(tr, cb)), (cb, t)


@pytest.mark.parametrize("bits,cb", [(4, "3inst"), (3, "3inst"), (2, "mcg"), (2.5, "mul1"), (6, "mul1"), (8, "3inst"), (1, "3inst"), (3.5, "mul1")])
@pytest.mark.parametrize("rows", [1, 7, 64, 200, 300])
def test_exl3_gemm_matches_fp32_reference(K, bits, cb, rows):
    k, n = 512, 384
    w, tr, _, _ = _mk(K, k, n, bits, cb, seed=int(bits * 2) + rows)
    wq = torch.from_numpy(exl3.unpack_f32(tr, cb)).cuda()
    g = torch.Generator(device="cpu").manual_seed(rows)
    xr = (torch.randn(rows, k, generator=g) * 0.5).to(torch.float16).cuda()
    ref = xr.float() @ wq
    status = K.new_status()
    for splits in (1, 3):
        part = torch.full((splits * rows * n,), float("nan"), device="cuda")
        K.exl3_gemm(xr, w, part, splits, status)
        torch.cuda.synchronize()
        K.check_status(status)
        got = part.view(splits, rows, n).sum(0)
        err = (got - ref).abs().max().item()
        assert err <= 2e-3 * ref.abs().max().item() + 1e-3, (bits, cb, rows, splits, err)


@pytest.mark.parametrize("cb", ["3inst", "mcg", "mul1"])
def test_exl3_gemm_4bpw_tensor_memory_path_equals_shared_memory_path(K, cb):
    """The 4.0 bpw kernel keeps decoded weights in tensor memory; same products, same K order -> same bits as the generic kernel."""
    k, n = 2048, 512     # 16 chunks per CTA at one split: every ring wraps several times
    w, tr, _, _ = _mk(K, k, n, 4, cb, seed=11)
    status = K.new_status()
    for rows in (1, 40, 64, 130, 520):
        xr = (torch.randn(rows, k) * 0.5).to(torch.float16).cuda()
        a = torch.zeros(2 * rows * n, device="cuda")
        b = torch.zeros(2 * rows * n, device="cuda")
        ref = xr.float() @ torch.from_numpy(exl3.unpack_f32(tr, cb)).cuda()
        for splits in (2, 1):
            a.zero_(); b.zero_()
            K.exl3_gemm(xr, w, a, splits, status)
            K.exl3_gemm(xr, w, b, splits, status, force_generic=True)
            torch.cuda.synchronize()
            K.check_status(status)
            assert (a.view(2, rows, n)[:splits].sum(0) - ref).abs().max() <= 2e-3 * ref.abs().max() + 1e-3
            assert torch.equal(a, b), (rows, splits)


def test_exl3_gemm_row_invariance(K):
    """A row's bits do not depend on the other rows or their count (decode class)."""
    k, n = 1024, 256
    w, _, _, _ = _mk(K, k, n, 4, seed=3)
    xr = (torch.randn(64, k) * 0.5).to(torch.float16).cuda()
    status = K.new_status()
    outs = []
    for rows in (1, 5, 16, 33, 64):
        part = torch.zeros(2 * rows * n, device="cuda")
        K.exl3_gemm(xr[:rows].contiguous(), w, part, 2, status)
        outs.append(part.view(2, rows, n)[:, 0].clone())
    torch.cuda.synchronize()
    K.check_status(status)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


def _hadamard(x):
    h = torch.from_numpy(exl3.hadamard128(np.float32)).to(x.device)
    return (x.reshape(*x.shape[:-1], -1, 128) @ h).reshape(x.shape)


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def test_norm_rot_in_and_finish_kernels(K):
    torch.manual_seed(0)
    M, d, F, S, eps = 5, 512, 256, 3, 1e-6
    x = torch.randn(M, d).to(torch.bfloat16).cuda()
    nw = (1 + 0.1 * torch.randn(d)).to(torch.bfloat16).cuda()
    suh = (torch.rand(d) + 0.5).to(torch.float16).cuda()
    xr = torch.empty(M, d, dtype=torch.float16, device="cuda")
    K.norm_rot_in(x, nw, eps, suh, xr)
    ref = _hadamard(_rms(x.float(), 1.0, eps).to(torch.bfloat16).float() * nw.float() * suh.float())
    assert (xr.float() - ref).abs().max() < 2e-2
    K.norm_rot_in(x, None, eps, suh, xr)
    assert (xr.float() - _hadamard(x.float() * suh.float())).abs().max() < 2e-2
    # finish_store
    w, _, _, svh = _mk(K, 128, d, 4)
    part = torch.randn(S, M, d, device="cuda")
    y_ref = _hadamard(part.sum(0)) * w.svh.float()
    out = torch.empty(M, d, dtype=torch.float32, device="cuda")
    K.finish_store(part, S, M, w, out)
    assert (out - y_ref).abs().max() < 1e-4 * y_ref.abs().max() + 1e-5
    outb = torch.empty(M, d, dtype=torch.bfloat16, device="cuda")
    K.finish_store(part, S, M, w, outb)
    assert (outb.float() - y_ref).abs().max() < 1e-2 * y_ref.abs().max()
    # finish_add_norm_rot
    h = torch.randn(M, d).to(torch.bfloat16).cuda()
    h0 = h.clone()
    K.finish_add_norm_rot(part, S, M, w, h, nw, eps, suh, xr)
    h_ref = (h0.float() + y_ref).to(torch.bfloat16)
    assert (h.float() - h_ref.float()).abs().max() <= 0.04
    ref = _hadamard(_rms(h.float(), 1.0, eps).to(torch.bfloat16).float() * nw.float() * suh.float())
    assert (xr.float() - ref).abs().max() < 3e-2
    # finish_swiglu_rot
    wgu, _, _, _ = _mk(K, 128, 2 * F, 4, out_scale=0.5)
    partg = torch.randn(S, M, 2 * F, device="cuda")
    yg = _hadamard(partg.sum(0)) * wgu.svh.float()
    act = (torch.nn.functional.silu(yg[:, :F]) * yg[:, F:]).to(torch.bfloat16).float()
    sd = (torch.rand(F) + 0.5).to(torch.float16).cuda()
    xf = torch.empty(M, F, dtype=torch.float16, device="cuda")
    K.finish_swiglu_rot(partg, S, M, wgu, sd, xf)
    ref = _hadamard(act * sd.float())
    assert (xf.float() - ref).abs().max() < 2e-2 * max(1.0, ref.abs().max().item())


def test_topk_exact_order(K):
    torch.manual_seed(1)
    rows, vocab, count = 3, 151936, 28
    logits = torch.randn(rows, vocab, device="cuda")
    logits[0, 5] = logits[0, 77777] = 9.0  # tie -> lower id first
    scratch = K.topk_scratch(rows, vocab, count)
    ids = torch.empty(rows, count, dtype=torch.int32, device="cuda")
    vals = torch.empty(rows, count, dtype=torch.float32, device="cuda")
    K.topk(logits, count, scratch, ids, vals)
    v, i = torch.sort(logits, dim=1, descending=True, stable=True)
    assert torch.equal(vals, v[:, :count])
    assert ids[0, 0].item() == 5 and ids[0, 1].item() == 77777
    assert torch.equal(ids[1:].long(), i[1:, :count])


def _ref_attn(q, kc, vc, ctx, n_q, n_kv, hd):
    # q [n_q, hd]; kc, vc [T, n_kv, hd]
    g = n_q // n_kv
    k = kc[:ctx].float().repeat_interleave(g, dim=1)
    v = vc[:ctx].float().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,thd->ht", q.float(), k) / math.sqrt(hd)
    return torch.einsum("ht,thd->hd", torch.softmax(s, -1), v).reshape(-1)


@pytest.mark.parametrize("hd,n_q,n_kv", [(128, 10, 2), (64, 4, 2)])
def test_paged_attention_decode_and_prefill(K, hd, n_q, n_kv):
    torch.manual_seed(2)
    pages, nseq, max_blocks = 40, 3, 12
    kc = torch.zeros(pages, n_kv, 64, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    lens = [700, 65, 1]
    perm = torch.randperm(pages).tolist()
    bt = torch.zeros(nseq, max_blocks, dtype=torch.int32)
    seq_k, seq_v = [], []
    for s, T in enumerate(lens):
        k = torch.randn(T, n_kv, hd).to(torch.bfloat16)
        v = torch.randn(T, n_kv, hd).to(torch.bfloat16)
        seq_k.append(k.cuda()); seq_v.append(v.cuda())
        for b in range((T + 63) // 64):
            pg = perm.pop()
            bt[s, b] = pg
            n = min(64, T - b * 64)
            kc[pg, :, :n] = k[b * 64:b * 64 + n].transpose(0, 1).cuda()
            vc[pg, :, :n] = v[b * 64:b * 64 + n].transpose(0, 1).cuda()
    bt = bt.cuda()
    tk, tv = K.KvTensorMap(kc), K.KvTensorMap(vc)
    status = K.new_status()
    # decode: rows = last token of each sequence + one mid-sequence row (verify-window style)
    row_seq = torch.tensor([0, 1, 2, 0], dtype=torch.int32, device="cuda")
    ctx = torch.tensor([700, 65, 1, 300], dtype=torch.int32, device="cuda")
    q = torch.randn(4, n_q * hd).to(torch.bfloat16).cuda()
    scratch = K.attn_decode_scratch(4, n_q, hd, max_blocks * 64)
    out = torch.empty(4, n_q * hd, dtype=torch.bfloat16, device="cuda")
    suh = (torch.rand(n_q * hd) + 0.5).to(torch.float16).cuda()
    xr = torch.empty(4, n_q * hd, dtype=torch.float16, device="cuda")
    K.attn_decode(tk, tv, q, bt, row_seq, ctx, scratch, n_q, n_kv, hd, max_blocks * 64, 1 / math.sqrt(hd), suh, xr, out, status)
    torch.cuda.synchronize()
    K.check_status(status)
    for r in range(4):
        s = int(row_seq[r])
        ref = _ref_attn(q[r].view(n_q, hd), seq_k[s], seq_v[s], int(ctx[r]), n_q, n_kv, hd)
        assert (out[r].float() - ref).abs().max() < 2e-2, r
        assert (xr[r].float() - _hadamard(out[r].float() * suh.float())).abs().max() < 2e-2
    # verify window: rows that share a sequence are blocked into one CTA's MMA tile; every row's bits must equal the bits it gets alone
    wseq = [0, 0, 0, 0, 0, 1, 1, 0, 2]
    wctx = [252, 253, 254, 255, 256 + 1, 64, 65, 700, 1]
    W = len(wseq)
    qw = torch.randn(W, n_q * hd).to(torch.bfloat16).cuda()
    scr_w = K.attn_decode_scratch(W, n_q, hd, max_blocks * 64)
    out_w = torch.empty(W, n_q * hd, dtype=torch.bfloat16, device="cuda")
    xr_w = torch.empty(W, n_q * hd, dtype=torch.float16, device="cuda")
    outs = []
    for msr in (1, 5, 9):        # one, two and three MMA tiles per CTA: the same bits
        K.attn_decode(tk, tv, qw, bt, torch.tensor(wseq, dtype=torch.int32, device="cuda"), torch.tensor(wctx, dtype=torch.int32, device="cuda"),
                      scr_w, n_q, n_kv, hd, max_blocks * 64, 1 / math.sqrt(hd), suh, xr_w, out_w, status, max_seq_rows=msr)
        torch.cuda.synchronize()
        K.check_status(status)
        outs.append((out_w.clone(), xr_w.clone()))
    assert all(torch.equal(o, outs[0][0]) and torch.equal(x, outs[0][1]) for o, x in outs[1:])
    scr_1 = K.attn_decode_scratch(1, n_q, hd, max_blocks * 64)
    for r in range(W):
        out_1 = torch.empty(1, n_q * hd, dtype=torch.bfloat16, device="cuda")
        xr_1 = torch.empty(1, n_q * hd, dtype=torch.float16, device="cuda")
        K.attn_decode(tk, tv, qw[r:r + 1].contiguous(), bt, torch.tensor(wseq[r:r + 1], dtype=torch.int32, device="cuda"),
                      torch.tensor(wctx[r:r + 1], dtype=torch.int32, device="cuda"), scr_1, n_q, n_kv, hd, max_blocks * 64, 1 / math.sqrt(hd),
                      suh, xr_1, out_1, status)
        torch.cuda.synchronize()
        assert torch.equal(out_w[r], out_1[0]) and torch.equal(xr_w[r], xr_1[0]), r
        ref = _ref_attn(qw[r].view(n_q, hd), seq_k[wseq[r]], seq_v[wseq[r]], wctx[r], n_q, n_kv, hd)
        assert (out_w[r].float() - ref).abs().max() < 2e-2, r
    # prefill: sequence 0 rows 500..699 (chunk of 200) and sequence 1 whole (65 rows)
    q_start = torch.tensor([0, 200], dtype=torch.int32, device="cuda")
    q_len = torch.tensor([200, 65], dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([500, 0], dtype=torch.int32, device="cuda")
    seq_ids = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    qp = torch.randn(265, n_q * hd).to(torch.bfloat16).cuda()
    outp = torch.zeros(265, n_q * hd, dtype=torch.bfloat16, device="cuda")
    K.attn_prefill(tk, tv, qp, bt, seq_ids, q_start, q_len, pos0, outp, 2, 200, n_q, n_kv, hd, 1 / math.sqrt(hd), status)
    torch.cuda.synchronize()
    K.check_status(status)
    for r in list(range(0, 200, 37)) + [199, 200, 230, 264]:
        s, p = (0, 500 + r) if r < 200 else (1, r - 200)
        ref = _ref_attn(qp[r].view(n_q, hd), seq_k[s], seq_v[s], p + 1, n_q, n_kv, hd)
        assert (outp[r].float() - ref).abs().max() < 2e-2, r


def test_qkv_finish_rope_and_cache_write(K):
    torch.manual_seed(3)
    M, n_q, n_kv, hd, S = 3, 4, 2, 128, 2
    N = (n_q + 2 * n_kv) * hd
    w, _, _, _ = _mk(K, 128, N, 4, out_scale=1.0)
    part = torch.randn(S, M, N, device="cuda")
    y = _hadamard(part.sum(0)) * w.svh.float()
    pos = torch.tensor([0, 17, 4099], dtype=torch.int32, device="cuda")
    slot = torch.tensor([64 * 3 + 0, 64 * 1 + 17, -1], dtype=torch.int32, device="cuda")
    inv = torch.from_numpy((1.0 / (1e4 ** (np.arange(0, hd, 2, dtype=np.float32) / hd))).astype(np.float32)).cuda()
    kc = torch.zeros(5, n_kv, 64, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qo = torch.empty(M, n_q * hd, dtype=torch.bfloat16, device="cuda")
    K.finish_qkv_rope(part, S, M, n_q, n_kv, hd, w, None, None, 1e-6, pos, inv, slot, qo, kc, vc)

    def rope(x, p):
        ang = p.float()[:, None] * inv[None]
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    qr = rope(y[:, :n_q * hd].view(M, n_q, hd), pos).reshape(M, -1)
    kr = rope(y[:, n_q * hd:(n_q + n_kv) * hd].view(M, n_kv, hd), pos)
    v = y[:, (n_q + n_kv) * hd:].view(M, n_kv, hd)
    assert (qo.float() - qr).abs().max() < 3e-2 * qr.abs().max()
    assert (kc[3, :, 0].float() - kr[0]).abs().max() < 3e-2 * kr.abs().max()
    assert (kc[1, :, 17].float() - kr[1]).abs().max() < 3e-2 * kr.abs().max()
    assert (vc[1, :, 17].float() - v[1]).abs().max() < 3e-2 * v.abs().max()
    assert kc[0].abs().max() == 0 and kc[2].abs().max() == 0 and kc[4].abs().max() == 0


def test_interleaved_mrope_matches_reference_and_reduces_to_rope(K):
    """Frequency pair i rotates by the T, H or W position (axis i % 3 inside its section); equal axes give plain RoPE bit for bit."""
    torch.manual_seed(7)
    M, n_q, n_kv, hd = 6, 4, 2, 128
    N = (n_q + 2 * n_kv) * hd
    w, _, _, _ = _mk(K, 128, N, 4, out_scale=1.0)
    part = torch.randn(1, M, N, device="cuda")
    y = _hadamard(part.sum(0)) * w.svh.float()
    inv = torch.from_numpy((1.0 / (1e4 ** (np.arange(0, hd, 2, dtype=np.float32) / hd))).astype(np.float32)).cuda()
    sec = (24, 20, 20)
    pos3 = torch.tensor([[0, 0, 0], [5, 5, 5], [9, 2, 7], [9, 3, 1], [100, 40, 41], [4099, 0, 63]], dtype=torch.int32, device="cuda")
    slot = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    kc = torch.zeros(2, n_kv, 64, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)

    def run(p3, positions):
        qo = torch.empty(M, n_q * hd, dtype=torch.bfloat16, device="cuda")
        K.finish_qkv_rope(part, 1, M, n_q, n_kv, hd, w, None, None, 1e-6, positions, inv, slot, qo, kc, vc, pos3=p3, mrope_sections=sec if p3 is not None else None)
        return qo
    t_only = pos3[:, 0].contiguous()
    same = t_only[:, None].repeat(1, 3).contiguous()
    assert torch.equal(run(same, t_only), run(None, t_only))
    got = run(pos3, t_only).float().view(M, n_q, hd)
    i = torch.arange(hd // 2, device="cuda")
    axis = torch.where((i % 3 == 1) & (i < 3 * sec[1]), 1, torch.where((i % 3 == 2) & (i < 3 * sec[2]), 2, 0))
    p = pos3.float()[:, axis]                                    # [M, hd/2]
    ang = p * inv[None]
    c, s_ = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
    x = y[:, :n_q * hd].view(M, n_q, hd)
    x1, x2 = x[..., :hd // 2], x[..., hd // 2:]
    ref = torch.cat([x1 * c - x2 * s_, x2 * c + x1 * s_], -1)
    assert (got - ref).abs().max() < 3e-2 * ref.abs().max()
    assert (got[2] - run(None, t_only).float().view(M, n_q, hd)[2]).abs().max() > 0.1        # the H / W axes really rotate differently


def test_state_digest_equals_the_host_digest_and_sees_every_byte(K):
    torch.manual_seed(3)
    for n in (8, 24, 4096, 1_000_003):
        t = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
        d = K.state_digest(t)
        want = K.state_digest_host(bytes(t.cpu().numpy()))
        assert (int(d[0].item()) & 0xFFFFFFFFFFFFFFFF) == want, n
    a = torch.randn(3, 1000, device="cuda")
    b = a.clone()
    b[2, 999] += 1e-3
    swapped = a.flip(0).contiguous()
    da, db, ds = (int(K.state_digest(x)[0].item()) for x in (a, b, swapped))
    assert da != db and da != ds                                   # one changed value, and the same rows in another order
    parts = K.state_digest([a, b]).cpu().tolist()
    assert K.fold_digest(parts) != K.fold_digest(parts[::-1])


def _hc_reference(x, fn, base, scales, norm_w, y, rms_eps, hc_eps, norm_eps, iters):
    """Plain float64 form of one hyper-connection site: (coef [rows, 24], sublayer input [rows, D], streams after the apply)."""
    x, fn, base, norm_w, y = (t.double() for t in (x, fn, base, norm_w, y))
    rows, ns, D = x.shape
    flat = x.reshape(rows, ns * D)
    S = flat @ fn.T
    rmr = 1.0 / torch.sqrt((flat * flat).sum(1, keepdim=True) / (ns * D) + rms_eps)
    pre = torch.sigmoid(S[:, :4] * rmr * scales[0] + base[:4]) + hc_eps
    post = 2 * torch.sigmoid(S[:, 4:8] * rmr * scales[1] + base[4:8])
    c = torch.softmax((S[:, 8:] * rmr * scales[2] + base[8:]).view(rows, 4, 4), dim=2) + hc_eps
    c = c / (c.sum(1, keepdim=True) + hc_eps)
    for _ in range(iters - 1):
        c = c / (c.sum(2, keepdim=True) + hc_eps)
        c = c / (c.sum(1, keepdim=True) + hc_eps)
    col = (pre[:, :, None] * x).sum(1)
    hn = col / torch.sqrt((col * col).mean(1, keepdim=True) + norm_eps) * norm_w
    new = post[:, :, None] * y[:, None, :] + torch.einsum("rgh,rgd->rhd", c, x)
    return torch.cat([pre, post, c.reshape(rows, 16)], 1), hn, new


def test_hyper_connection_mix_and_apply_match_the_reference_and_are_row_invariant(K):
    torch.manual_seed(11)
    for D in (512, 5120):
        rows = 7
        x = torch.randn(rows, 4, D, device="cuda")
        fn = torch.randn(24, 4 * D, device="cuda") / math.sqrt(4 * D)
        base = torch.randn(24, device="cuda") * 0.5
        scales = (0.7, 1.3, 2.0)
        nw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
        y = torch.randn(rows, D, device="cuda")
        coef = torch.empty(rows, 24, device="cuda")
        hn = torch.empty(rows, D, dtype=torch.bfloat16, device="cuda")
        K.hc_mix(x, fn, base, scales, nw, coef, hn, iters=20)
        want_c, want_h, want_x = _hc_reference(x, fn, base, scales, nw.float(), y, 1e-6, 1e-6, 1e-6, 20)
        assert (coef.double() - want_c).abs().max() < 1e-4
        comb = coef[:, 8:].view(rows, 4, 4)
        assert (comb.sum(1) - 1).abs().max() < 1e-3 and (comb.sum(2) - 1).abs().max() < 1e-2          # Sinkhorn: (almost) doubly stochastic
        assert (hn.double() - want_h).abs().max() < 2e-2 * want_h.abs().max()
        x2 = x.clone()
        K.hc_apply(x2, y, coef)
        assert (x2.double() - want_x).abs().max() < 1e-4 * want_x.abs().max() + 1e-4
        # a row's bits do not depend on the other rows of the launch
        c1 = torch.empty(1, 24, device="cuda")
        h1 = torch.empty(1, D, dtype=torch.bfloat16, device="cuda")
        K.hc_mix(x[3:4].contiguous(), fn, base, scales, nw, c1, h1, iters=20)
        assert torch.equal(c1[0], coef[3]) and torch.equal(h1[0], hn[3])


@pytest.mark.parametrize("rows,K,N", [(1, 512, 256), (5, 1024, 384), (70, 2048, 256), (300, 512, 128)])
def test_fp8_block_scaled_linear_matches_fp32(rows, K, N):
    """E4M3 weights with one power-of-two scale per 32 x 32 tile on the tcgen05 kernel against x @ dequant(W)^T in fp32; a row's bits do not
    depend on the rows it shares the launch with or on its place among them (same K splits, same tile class)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(rows + K)
    dense = torch.randn(N, K, device="cuda", generator=g) * torch.exp2(torch.randint(-6, 5, (N // 32, 1, K // 32, 1), device="cuda", generator=g).float()
                                                                      ).expand(N // 32, 32, K // 32, 32).reshape(N, K)
    bias = torch.randn(N, device="cuda", generator=g)
    w = K_.Fp8Weight.quantize(dense, bias)
    x = torch.randn(rows, K, device="cuda", generator=g).to(torch.bfloat16)
    status = K_.new_status()
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        got = K_.fp8_linear(x, w, status, out_dtype=dt)
        torch.cuda.synchronize()
        K_.check_status(status)
        want = x.float() @ w.dense().T + bias
        tol = 1e-4 if dt == torch.float32 else 1e-2
        assert torch.allclose(got.float(), want, rtol=tol, atol=tol * want.abs().max().item()), dt
    if rows > 1:      # the same rows one position earlier in a launch of the same tile class: bit-identical
        splits = 2
        full = K_.fp8_linear(x, w, status, out_dtype=torch.float32, splits=splits).clone()
        part = K_.fp8_linear(x[1:].contiguous(), w, status, out_dtype=torch.float32, splits=splits)
        torch.cuda.synchronize()
        K_.check_status(status)
        assert torch.equal(full[1:], part)
    y = K_.bf16_linear(x, dense.to(torch.bfloat16), bias.to(torch.bfloat16))
    assert torch.allclose(y.float(), x.float() @ dense.to(torch.bfloat16).float().T + bias.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2 * y.abs().max().item())


def test_long_k_pipelines_are_exact_and_repeatable():
    """32 and 64 K chunks per CTA with 128-row tiles, integer-valued data (every fp32 sum is exact, so any difference is a wrong byte, not a
    rounding order): the FP8 linear and the MXFP4 expert GEMM give the exact product on every one of many back-to-back launches.  (Each stage of
    their weight rings is read with ordinary loads and refilled by a bulk tensor copy; the release needs a proxy fence, without which the copy
    overtook the reads in about half of such launches.)"""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.format import mxfp4
    from rexl3_b200.ops import kernels as K_
    from rexl3_b200.ops import lib as L
    lib = L.load()
    g = torch.Generator(device="cuda").manual_seed(1)
    st = K_.new_status()
    N, Kd, rows = 256, 2048, 70
    xi = torch.randint(-2, 3, (rows, Kd), device="cuda", generator=g).to(torch.bfloat16)
    wi = K_.Fp8Weight.quantize(torch.randint(-3, 4, (N, Kd), device="cuda", generator=g).float())
    want = xi.float() @ wi.dense().T
    bad = sum(int(not torch.equal(K_.fp8_linear(xi, wi, st, out_dtype=torch.float32, splits=1), want)) for _ in range(30))
    K_.check_status(st)
    assert bad == 0
    rng = np.random.default_rng(1)
    Kd = 4096
    q, s = mxfp4.quantize(rng.normal(0, 0.05, size=(N, Kd)).astype(np.float32))
    wf = torch.from_numpy(mxfp4.dequant(q, s)).cuda()
    d_w, d_s = torch.from_numpy(q.view(np.uint8)[None].copy()).cuda(), torch.from_numpy(s[None].copy()).cuda()
    xs = torch.from_numpy(rng.integers(-2, 3, size=(rows, Kd)).astype(np.float32)).cuda().to(torch.float16)
    tile_tab = torch.tensor([0, 0, rows], dtype=torch.int32, device="cuda")
    want = xs.float() @ wf.T
    bad = 0
    for _ in range(30):
        part = torch.zeros(1, rows, N, dtype=torch.float32, device="cuda")
        L.check(lib.rx_mxfp4_gemm_grouped(xs.data_ptr(), rows, Kd, d_w.data_ptr(), d_s.data_ptr(), 1, N, part.data_ptr(), 1, tile_tab.data_ptr(), 1, 128,
                                          st.data_ptr(), L.stream_ptr()), "mxfp4")
        bad += int(not torch.equal(part[0], want))
    K_.check_status(st)
    assert bad == 0
