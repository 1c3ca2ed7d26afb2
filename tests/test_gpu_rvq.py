"""Residual vector quantisation on the GPU (tensor-core pre-selection + exact FP32 decision, ordered decode)
vs the reference's codes (golden fixture) and the CPU oracle."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from conftest import load_golden, rvq_recipe
from oracle import mimi_attention_oracle as O

pytestmark = pytest.mark.gpu


def _books(embed_sum, usage):
    return embed_sum / usage.clamp(min=1e-5)[:, :, None]


def test_rvq_codes_match_the_reference_fixture():
    import fast_mimi_b200 as fm
    g = load_golden("rvq_codes.npz")
    gen, embed_sum, usage, proj = rvq_recipe(31, 7)
    emb = torch.randn(2, 512, 40, generator=gen) * 3
    books = _books(embed_sum, usage)
    x = F.conv1d(emb, proj[:, :, None]).permute(0, 2, 1).reshape(-1, 256)
    gb = fm.ops.RVQCodebooks(books.cuda())
    codes, cand = fm.ops.rvq_encode(x.cuda(), gb, return_candidates=True)
    assert torch.equal(codes.cpu().view(7, 2, 40), g["codes"])
    assert int(cand.min()) >= 1 and float(cand.float().mean()) < 16       # a handful of exact evaluations per frame
    for dt in (torch.float16, torch.float32):                               # the forms with the scores in memory
        assert torch.equal(fm.ops.rvq_encode(x.cuda(), gb, scores_dtype=dt).cpu().view(7, 2, 40), g["codes"])
    dec = fm.ops.rvq_decode(codes, gb).cpu().view(2, 40, 256).permute(0, 2, 1)
    assert torch.equal(dec[:, :, ::13], g["quantized_probe"])             # ordered FP32 adds: bit-exact


@pytest.mark.parametrize("scores_dtype", [None, torch.float16, torch.float32])      # None: candidate records, no scores in memory
@pytest.mark.parametrize("rows,layers", [(1, 8), (257, 3), (6000, 8)])
def test_rvq_codes_match_the_oracle(rows, layers, scores_dtype):
    """Frame-level identity (all layers' codes equal) against the CPU oracle; inputs scaled so that the later
    layers see residuals two orders of magnitude smaller than the first."""
    import fast_mimi_b200 as fm
    gen, embed_sum, usage, _ = rvq_recipe(rows, layers)
    books = _books(embed_sum, usage)
    books = books * (0.5 ** torch.arange(layers, dtype=torch.float32))[:, None, None]    # finer codebooks deeper down
    x = torch.randn(rows, 256, generator=gen) * 1.5
    want = O.rvq_encode(x, books)
    gb = fm.ops.RVQCodebooks(books.cuda())
    got = fm.ops.rvq_encode(x.cuda(), gb, scores_dtype=scores_dtype).cpu()
    frames_same = int((got == want).all(dim=0).sum())
    # Where a frame differs, the two nearest entries are closer together than FP32 rounding resolves: the oracle
    # (like the reference) takes argmin over torch.cdist, which for more than 25 rows evaluates |x|^2 + |e|^2 - 2 x.e
    # through a matrix product, the kernel decides by sum_k (x_k - e_k)^2.  An FP64 evaluation of the exact
    # distances says which of the two is nearer to the truth at the first layer where they part.
    first_diff = (got != want).int().argmax(dim=0)
    differing = ((got != want).any(dim=0)).nonzero().flatten().tolist()
    ours_better = 0
    for r in differing:
        l = int(first_diff[r])
        resid = x[r].double()
        for j in range(l):
            resid = resid - books[j, got[j, r]].double()
        d = ((resid[None] - books[l].double()) ** 2).sum(-1)
        ours_better += int(d[got[l, r]] <= d[want[l, r]])
    print(f"rvq rows={rows} layers={layers} scores={scores_dtype}: {frames_same} of {rows} frames have all codes equal to "
          f"the oracle's; of the {len(differing)} others the kernel's choice is the nearer one in FP64 for {ours_better}")
    assert frames_same >= 0.995 * rows, frames_same
    assert torch.equal(fm.ops.rvq_decode(got.cuda(), gb).cpu(), O.rvq_decode(got, books))


@pytest.mark.parametrize("rows,n,k", [(1000, 256, 512), (64, 512, 256), (4099, 256, 512)])
def test_split_precision_linear_has_fp32_accuracy(rows, n, k):
    """The quantiser's input / output projections on the FP16 tensor core (hi + lo parts, FP32 accumulation) against
    an FP64 product and against the FP32 verification kernel."""
    import fast_mimi_b200 as fm
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, k, generator=g) * 3).cuda()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).cuda()
    got = fm.ops.linear_split(x, fm.ops.split_half(w))
    ref64 = (x.double() @ w.double().T)
    err = float((got.double() - ref64).abs().max() / ref64.abs().max())
    err32 = float((fm.ops.linear_fp32(x, w).double() - ref64).abs().max() / ref64.abs().max())
    print(f"split-precision linear {rows}x{k}->{n}: max error / max |y| = {err:.2e} (FP32 CUDA-core kernel: {err32:.2e})")
    assert err < 2e-6 and err < 2 * err32 + 1e-7       # as good as an FP32 product of the same operands


def test_non_finite_residual_is_reported_not_quantised():
    import fast_mimi_b200 as fm
    gb = fm.ops.RVQCodebooks(torch.randn(1, 256, 256).cuda())
    x = torch.randn(4, 256).cuda()
    x[2, 7] = float("nan")
    st = fm.ops.new_status("cuda")
    fm.ops.rvq_encode(x, gb, status=st)
    assert fm.ops.read_status(st) == 105
    with pytest.raises(RuntimeError, match="105"):
        fm.check_status(status=st)


def test_rvq_decode_rejects_out_of_range_codes():
    import fast_mimi_b200 as fm
    gb = fm.ops.RVQCodebooks(torch.randn(2, 256, 256).cuda())
    codes = torch.tensor([[0, 5], [256, 1]], dtype=torch.int64).cuda()
    with pytest.raises(RuntimeError):
        fm.ops.rvq_decode(codes, gb)


def test_split_quantizer_wrapper_matches_oracle_encode_and_decode():
    """MimiSplitRVQB200 built from modules that carry the reference's attribute names (layers[i].codebook.embed,
    1 x 1 input_proj / output_proj): encode codes and decode output against the oracle with the same projections."""
    import types
    import torch.nn as nn
    import fast_mimi_b200 as fm

    def branch(seed, layers):
        gen, embed_sum, usage, proj = rvq_recipe(seed, layers)
        books = _books(embed_sum, usage)
        mod = types.SimpleNamespace()
        mod.layers = [types.SimpleNamespace(codebook=types.SimpleNamespace(embed=books[i].cuda())) for i in range(layers)]
        mod.input_proj = nn.Conv1d(512, 256, 1, bias=False)
        mod.output_proj = nn.Conv1d(256, 512, 1, bias=False)
        with torch.no_grad():
            mod.input_proj.weight.copy_(proj[:, :, None])
            mod.output_proj.weight.copy_(torch.randn(512, 256, 1, generator=gen) / 16)
        mod.input_proj.cuda(); mod.output_proj.cuda()
        return mod, books

    sem, sem_books = branch(41, 1)
    aco, aco_books = branch(42, 7)
    split = types.SimpleNamespace(semantic_residual_vector_quantizer=sem, acoustic_residual_vector_quantizer=aco)
    native = fm.MimiSplitRVQB200.from_reference(split)
    emb = torch.randn(3, 512, 50, generator=torch.Generator().manual_seed(43)) * 3

    def oracle_encode(mod, books, n):
        x = F.conv1d(emb, mod.input_proj.weight.cpu()).permute(0, 2, 1).reshape(-1, 256)
        return O.rvq_encode(x, books, n).view(n, 3, 50)

    want = torch.cat((oracle_encode(sem, sem_books, 1), oracle_encode(aco, aco_books, 7)))
    got = native.encode(emb.cuda(), 8).cpu()
    assert got.shape == (8, 3, 50)
    same = int((got == want).all(dim=0).sum())
    print(f"split quantiser wrapper: {same} of 150 frames have all 8 codes equal to the oracle's")
    assert same >= 0.995 * 150
    assert torch.equal(native.encode(emb.cuda(), 3).cpu(), got[:3])

    codes = got.permute(1, 0, 2).contiguous()                       # [B, K, T] as the reference's decode takes them
    dec = native.decode(codes.cuda()).cpu()

    def oracle_decode(mod, books, c):                               # c [K, B*T]
        q = O.rvq_decode(c, books).view(3, 50, 256).permute(0, 2, 1)
        return F.conv1d(q, mod.output_proj.weight.cpu())

    flat = got.reshape(8, -1)
    ref = oracle_decode(sem, sem_books, flat[:1]) + oracle_decode(aco, aco_books, flat[1:])
    assert dec.shape == (3, 512, 50)
    assert O.rel_l2(dec, ref) < 1e-5
    with pytest.raises(ValueError):
        native.encode(emb.cuda(), 0)
