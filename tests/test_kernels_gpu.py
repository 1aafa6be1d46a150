"""Each kernel alone against a plain PyTorch float64 restatement of the same operation, at sizes other
than the engine's tiny models use: widths and vocabularies that are no power of two, head sizes in
steps of 16, odd numbers of heads and groups, ragged batches, page edges, windows."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOLERANCE = {torch.float32: dict(rtol=2e-5, atol=2e-6), torch.bfloat16: dict(rtol=2e-2, atol=2e-3)}


@pytest.fixture(scope="module")
def ops():
    from lalamo_b200 import ops as module

    module.configure_matmul_precision()
    return module


def dev(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.to("cuda").contiguous()


def rnd(tensor: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Rounds through the activation type, in float64."""
    return tensor.to(dtype).to(torch.float64)


def close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, scale: float = 1.0) -> None:
    tolerance = TOLERANCE[dtype]
    torch.testing.assert_close(got.double().cpu(), want.double(), rtol=tolerance["rtol"], atol=tolerance["atol"] * scale)


def status() -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("dim,vocab", [(80, 1000), (2048, 333)])
def test_embed(ops, dtype, dim, vocab):
    generator = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, dim, generator=generator).to(dtype)
    ids = torch.randint(0, vocab, (37,), generator=generator, dtype=torch.int32)
    out = torch.empty(37, dim, dtype=torch.float32, device="cuda")
    flag = status()
    ops.embed(dev(table), dev(ids), out, 1.5, flag)
    assert torch.equal(out.cpu(), table[ids.long()].float() * 1.5) and flag.item() == 0
    bad = ids.clone()
    bad[3] = vocab
    ops.embed(dev(table), dev(bad), out, 1.0, flag)
    assert flag.item() == 3  # reported, not read out of bounds


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("dim", [16, 80, 128, 384, 1000, 1152, 2048, 3968, 4096, 5120])  # multiples of 128 up to 4096: one warp per row
def test_rmsnorm(ops, dtype, dim):
    generator = torch.Generator().manual_seed(dim)
    rows = 19
    x = torch.randn(rows, dim, generator=generator) * 3
    delta = torch.randn(rows, dim, generator=generator).to(dtype)
    weight = 1 + 0.3 * torch.randn(dim, generator=generator)
    eps, offset = 1e-3, 0.25

    def reference(h: torch.Tensor) -> torch.Tensor:
        h = h.double()
        normed = rnd(h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps), dtype)
        return normed * rnd(weight.double() + offset, dtype)

    # 32-bit residual stream + delta, written back
    residual = dev(x.clone())
    out = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.rmsnorm(residual, dev(weight), out, eps, delta=dev(delta), scale_offset=offset, write_back=True)
    summed = x.double() + delta.double()
    close(out, reference(summed), dtype, scale=3)
    torch.testing.assert_close(residual.cpu().double(), summed, rtol=1e-6, atol=1e-6)
    # gathered rows, no write-back
    picks = torch.tensor([4, 0, 18, 4], dtype=torch.int32)
    out = torch.empty(4, dim, dtype=dtype, device="cuda")
    ops.rmsnorm(dev(x), dev(weight), out, eps, rows=dev(picks), scale_offset=offset)
    close(out, reference(x[picks.long()]), dtype, scale=3)
    # activation-typed input
    typed = x.to(dtype)
    out = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.rmsnorm(dev(typed), dev(weight), out, eps, scale_offset=offset)
    close(out, reference(typed), dtype, scale=3)


@pytest.mark.parametrize("dim,slices", [(192, 3), (1000, 2), (77, 5), (2048, 10)])
def test_rmsnorm_adds_a_product_left_in_slices(ops, dim, slices):
    """A product cut into K slices may be handed to the norm as its partial sums: the norm adds them in
    order and rounds the sum to bfloat16, exactly what summing first and adding the tensor gives."""
    generator = torch.Generator().manual_seed(dim + slices)
    rows, eps = 21, 1e-5
    x = torch.randn(rows, dim, generator=generator) * 3
    partials = torch.randn(slices, rows, dim, generator=generator)
    weight = 1 + 0.3 * torch.randn(dim, generator=generator)
    sliced = ops.SlicedSum(dev(partials), torch.bfloat16)
    total = torch.zeros(rows, dim)
    for part in partials:
        total = total + part  # float32, in slice order, as the kernels add
    delta = total.to(torch.bfloat16)
    torch.testing.assert_close(sliced.sum().cpu(), delta, rtol=0, atol=0)
    # through the norm, written back: bit-equal to the norm given the summed tensor
    first, second = dev(x.clone()), dev(x.clone())
    out_first = torch.empty(rows, dim, dtype=torch.bfloat16, device="cuda")
    out_second = torch.empty_like(out_first)
    ops.rmsnorm(first, dev(weight), out_first, eps, delta=sliced, write_back=True)
    ops.rmsnorm(second, dev(weight), out_second, eps, delta=dev(delta), write_back=True)
    torch.testing.assert_close(out_first, out_second, rtol=0, atol=0)
    torch.testing.assert_close(first, second, rtol=0, atol=0)
    torch.testing.assert_close(first.cpu(), x + delta.float(), rtol=0, atol=0)
    # gathered rows
    picks = dev(torch.tensor([20, 3, 3, 0], dtype=torch.int32))
    out_first, out_second = torch.empty(4, dim, dtype=torch.bfloat16, device="cuda"), torch.empty(4, dim, dtype=torch.bfloat16, device="cuda")
    ops.rmsnorm(dev(x), dev(weight), out_first, eps, delta=sliced, rows=picks)
    ops.rmsnorm(dev(x), dev(weight), out_second, eps, delta=dev(delta), rows=picks)
    torch.testing.assert_close(out_first, out_second, rtol=0, atol=0)
    # added onto the stream without a norm
    stream = dev(x.clone())
    ops.residual_add(stream, sliced)
    torch.testing.assert_close(stream.cpu(), x + delta.float(), rtol=0, atol=0)


def test_feed_tokens_takes_the_last_token_of_marked_segments_from_the_device(ops):
    """Segments with a source row get their last token from the ids sampled on the device; the others,
    and every other token, stay as the host wrote them; a row outside the sampled ids is reported."""
    lengths = [3, 1, 5, 1, 2]
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32)
    token_ids = torch.arange(100, 100 + sum(lengths), dtype=torch.int32)
    source = torch.tensor([-1, 2, 0, -1, 1], dtype=torch.int32)
    sampled = torch.tensor([7, 8, 9], dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    on_device = dev(token_ids.clone())
    ops.feed_tokens(on_device, dev(torch.from_numpy(starts)), dev(torch.tensor(lengths, dtype=torch.int32)), dev(source), dev(sampled), status)
    expected = token_ids.clone()
    expected[3] = 9    # segment 1 (one token) <- row 2
    expected[8] = 7    # segment 2's last of five <- row 0
    expected[11] = 8   # segment 4's last of two <- row 1
    torch.testing.assert_close(on_device.cpu(), expected, rtol=0, atol=0)
    assert int(status.item()) == 0
    ops.feed_tokens(on_device, dev(torch.from_numpy(starts)), dev(torch.tensor(lengths, dtype=torch.int32)), dev(torch.tensor([-1, 3, -1, -1, -1], dtype=torch.int32)),
                    dev(sampled), status)
    assert int(status.item()) == 3   # a token that cannot be found: reported like a token outside the vocabulary
    torch.testing.assert_close(on_device.cpu(), expected, rtol=0, atol=0)


def test_rmsnorm_refuses_what_it_cannot_do(ops):
    x = torch.zeros(2, 60000, device="cuda")
    with pytest.raises(ops.KernelError, match="exceed"):
        ops.rmsnorm(x, torch.ones(60000, device="cuda"), torch.empty_like(x), 1e-5)
    with pytest.raises(ops.KernelError, match="CUDA device"):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), torch.zeros(2, 8), 1e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("hidden,activation", [(192, "silu"), (1000, "silu"), (77, "gelu")])
def test_gated_activation(ops, dtype, hidden, activation):
    fused = (torch.randn(23, 2 * hidden, generator=torch.Generator().manual_seed(1)) * 2).to(dtype)
    out = torch.empty(23, hidden, dtype=dtype, device="cuda")
    ops.gated_activation(dev(fused), out, activation)
    up, gate = fused[:, :hidden].double(), fused[:, hidden:].double()
    act = gate * torch.sigmoid(gate) if activation == "silu" else 0.5 * gate * (1 + torch.erf(gate / math.sqrt(2)))
    close(out, up * rnd(act, dtype), dtype, scale=4)


def reference_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary: int) -> torch.Tensor:
    angles = (positions.float()[:, None] * inv_freq[None, :]).double()  # float32 product, as the kernel forms it
    cos, sin = torch.cos(angles)[:, None, :], torch.sin(angles)[:, None, :]
    half = rotary // 2
    first, second, tail = x[..., :half], x[..., half:rotary], x[..., rotary:]
    return torch.cat([first * cos - second * sin, second * cos + first * sin, tail], dim=-1)


def paged_setup(segments: list[tuple[int, int]], page_size: int, generator: torch.Generator):
    """segments: (context before, new tokens).  Pages are handed out in a scrambled order."""
    blocks = [-(-(context + new) // page_size) for context, new in segments]
    total = sum(blocks)
    order = torch.randperm(total + 3, generator=generator).tolist()
    table = torch.full((len(segments), max(blocks)), -1, dtype=torch.int32)
    cursor = 0
    for row, count in enumerate(blocks):
        table[row, :count] = torch.tensor(order[cursor : cursor + count], dtype=torch.int32)
        cursor += count
    positions = torch.cat([torch.arange(c, c + n, dtype=torch.int32) for c, n in segments])
    token_segment = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, (_, n) in enumerate(segments)])
    return table, positions, token_segment, total + 3


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("many_tokens", [False, True], ids=["few", "many"])  # one warp per head / one block per token (scalar, or 16-byte for bfloat16 and head sizes 16 to 128 that are powers of two)
@pytest.mark.parametrize("heads,groups,head_dim,rotary,page_size,normed", [
    (5, 5, 48, 48, 16, True), (6, 2, 80, 32, 8, True), (3, 1, 128, 128, 64, False), (7, 1, 16, 0, 16, True),
    (9, 3, 64, 64, 16, True), (4, 2, 32, 16, 16, True), (7, 1, 16, 16, 32, True), (40, 8, 128, 64, 16, True),  # the 16-byte kernel for many tokens
])
def test_qk_norm_rope_write(ops, dtype, many_tokens, heads, groups, head_dim, rotary, page_size, normed):
    segments = [(0, 21), (37, 1), (page_size - 1, 3), (5000, 2)] + ([(200, 90)] if many_tokens else [])
    check_qk_norm_rope_write(ops, dtype, segments, heads, groups, head_dim, rotary, page_size, normed)


@pytest.mark.parametrize("heads,groups,head_dim,rotary,page_size,normed", [
    (9, 3, 64, 64, 16, True), (4, 2, 32, 16, 16, True), (7, 1, 16, 16, 32, True), (40, 8, 128, 64, 16, True), (3, 1, 128, 128, 64, False), (32, 8, 64, 64, 16, True),
])
def test_qk_norm_rope_write_in_runs(ops, heads, groups, head_dim, rotary, page_size, normed):
    """Hundreds of tokens: the kernel that takes four consecutive tokens per block and stores their values four rows at
    a time where they lie together.  Portions that start at a multiple of four in the batch and in their request
    (the first and the fourth), one that does not (the last), single tokens between them, a last run of two tokens."""
    segments = [(0, 300), (37, 1), (page_size - 1, 3), (8, 120), (203, 250)]
    assert sum(count for _, count in segments) % 4 == 2
    check_qk_norm_rope_write(ops, torch.bfloat16, segments, heads, groups, head_dim, rotary, page_size, normed)


def check_qk_norm_rope_write(ops, dtype, segments, heads, groups, head_dim, rotary, page_size, normed):
    generator = torch.Generator().manual_seed(heads * 100 + head_dim)
    table, positions, token_segment, num_pages = paged_setup(segments, page_size, generator)
    tokens = positions.numel()
    width = (heads + 2 * groups) * head_dim
    qkv = torch.randn(tokens, width, generator=generator).to(dtype)
    q_weight = (1 + 0.2 * torch.randn(head_dim, generator=generator)) if normed else None
    k_weight = (1 + 0.2 * torch.randn(head_dim, generator=generator)) if normed else None
    inv_freq = (1.0 / (torch.tensor(10000.0) ** (torch.arange(0, rotary, 2).float() / rotary))) if rotary else None
    eps = 1e-4
    k_pages = torch.full((num_pages, page_size, groups, head_dim), 99.0, dtype=dtype, device="cuda")
    v_pages = torch.full((num_pages, groups, head_dim, page_size), 99.0, dtype=dtype, device="cuda")
    q_out = torch.empty(tokens, heads * head_dim, dtype=dtype, device="cuda")
    flag = status()
    ops.qk_norm_rope_write(
        dev(qkv), q_out, k_pages, v_pages, q_weight=None if q_weight is None else dev(q_weight), k_weight=None if k_weight is None else dev(k_weight),
        eps=eps, scale_offset=0.0, inv_freq=None if inv_freq is None else dev(inv_freq), rotary_dim=rotary, positions=dev(positions),
        token_segment=dev(token_segment), block_table=dev(table), num_heads=heads, num_groups=groups, head_dim=head_dim, write_kv=True, status=flag)
    assert flag.item() == 0

    def transform(x: torch.Tensor, weight: torch.Tensor | None) -> torch.Tensor:
        x = x.double()
        if weight is not None:
            x = rnd(rnd(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps), dtype) * rnd(weight.double(), dtype), dtype)
        return reference_rope(x, positions, inv_freq, rotary) if rotary else x

    q = qkv[:, : heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim : (heads + groups) * head_dim].reshape(tokens, groups, head_dim)
    v = qkv[:, (heads + groups) * head_dim :].reshape(tokens, groups, head_dim)
    close(q_out.reshape(tokens, heads, head_dim), transform(q, q_weight), dtype, scale=3)
    k_expected, k_host, v_host = transform(k, k_weight), k_pages.cpu(), v_pages.cpu()
    written = torch.zeros(num_pages, page_size, dtype=torch.bool)
    for t in range(tokens):
        position, segment = int(positions[t]), int(token_segment[t])
        page, row = int(table[segment, position // page_size]), position % page_size
        close(k_host[page, row], k_expected[t], dtype, scale=3)
        assert torch.equal(v_host[page, :, :, row], v[t])  # values are stored transposed: [page, group, channel, row]
        written[page, row] = True
    assert (k_host[~written] == 99.0).all() and (v_host.permute(0, 3, 1, 2)[~written] == 99.0).all()  # nothing else was touched


def reference_attention(q, keys, values, position, scale, window):
    """One query [heads, hd] at `position` against keys/values [len, groups, hd] of its request."""
    heads, groups = q.shape[0], keys.shape[1]
    first = max(0, position - window + 1) if window else 0
    out = torch.zeros_like(q)
    for h in range(heads):
        g = h // (heads // groups)
        scores = (keys[first : position + 1, g] @ q[h]) * scale
        out[h] = torch.softmax(scores, dim=0) @ values[first : position + 1, g]
    return out


def call_attention(ops, kind, q, k_pages, v_pages, out, positions, token_segment, table, heads, groups, head_dim, scale, window, flag):
    common = dict(positions=dev(positions), token_segment=dev(token_segment), block_table=dev(table), num_heads=heads, num_groups=groups,
                  head_dim=head_dim, scale=scale, window=window, status=flag)
    if kind == "plain":
        ops.paged_attention_plain(q, k_pages, v_pages, out, **common)
    elif kind == "decode":
        ops.attention_decode(q, k_pages, v_pages, out, max_context=int(positions.max()) + 1, **common)
    elif kind == "decode_listed":  # only the listed tokens run; the others keep what out held
        listed = torch.arange(positions.numel() - 1, -1, -2, dtype=torch.int32)
        out.fill_(123.0)
        ops.attention_decode(q, k_pages, v_pages, out, max_context=int(positions.max()) + 1, token_list=dev(listed), num_listed=listed.numel(), **common)
        skipped = torch.ones(positions.numel(), dtype=torch.bool)
        skipped[listed.long()] = False
        assert (out[skipped.cuda()] == 123.0).all()
        rest = torch.nonzero(skipped).flatten().to(torch.int32)
        if rest.numel():
            ops.attention_decode(q, k_pages, v_pages, out, max_context=int(positions.max()) + 1, token_list=dev(rest), **common)
    else:  # "prefill", "prefill_mma", "prefill_tcgen05": tiles of at most 32 consecutive tokens of one request
        tiles, start = [], 0
        segments = token_segment.tolist()
        while start < len(segments):
            stop = start
            while stop < len(segments) and segments[stop] == segments[start] and stop - start < 32:
                stop += 1
            tiles.append((start, stop - start))
            start = stop
        records = torch.tensor(tiles, dtype=torch.int32)
        kernel, _, split = kind[8:].partition("_split")  # "prefill_tcgen05_split2": tiles of at least 2 key tiles are shared by two CTAs
        ops.attention_prefill(q, k_pages, v_pages, out, tiles=dev(records), num_tiles=len(tiles), kernel=kernel or None, split_tiles=int(split or 0), **common)


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("heads,groups,head_dim,page_size,window", [
    (4, 2, 16, 16, None), (6, 3, 32, 8, None), (5, 1, 48, 16, 33), (3, 3, 64, 64, None), (2, 1, 80, 16, 300),
    (8, 2, 128, 16, None), (2, 2, 256, 32, 17),
])
def test_paged_attention_plain(ops, dtype, heads, groups, head_dim, page_size, window):
    check_attention(ops, "plain", dtype, heads, groups, head_dim, page_size, window)


@pytest.mark.parametrize("heads,groups,head_dim,page_size,window", [
    (4, 2, 16, 16, None), (6, 3, 32, 16, None), (5, 1, 48, 16, 33), (3, 3, 64, 64, None), (2, 1, 80, 16, 300), (32, 8, 64, 16, None),
    (8, 2, 128, 32, None), (40, 2, 96, 16, 70), (7, 7, 112, 48, None), (20, 1, 32, 16, 16),
])
def test_attention_decode(ops, heads, groups, head_dim, page_size, window):
    """The split-key tensor-core kernel: every head size it takes, more than 16 query heads per K/V
    head, windows, pages of several 16-key blocks; rows it must not read hold NaN."""
    check_attention(ops, "decode", torch.bfloat16, heads, groups, head_dim, page_size, window)
    check_attention(ops, "decode_listed", torch.bfloat16, heads, groups, head_dim, page_size, window)


@pytest.mark.parametrize("heads,groups,head_dim,page_size,window", [
    (4, 2, 16, 16, None), (6, 3, 32, 16, None), (5, 1, 48, 16, 33), (3, 3, 64, 64, None), (2, 1, 80, 16, 300), (32, 8, 64, 16, None),
    (8, 2, 128, 32, None), (32, 2, 96, 16, 70), (7, 7, 112, 48, None), (24, 1, 32, 16, 16), (3, 1, 32, 16, 5),
])
def test_attention_prefill(ops, heads, groups, head_dim, page_size, window):
    """The tiled tensor-core kernel: tiles of 32, 8 and 1 tokens, contexts before the portion, windows
    shorter than a tile, up to 24 query heads per K/V head; rows it must not read hold NaN."""
    check_attention(ops, "prefill", torch.bfloat16, heads, groups, head_dim, page_size, window)


@pytest.mark.parametrize("context,splits", [(9000, 1), (2077, 1), (4096, 3), (33, 1)])
def test_attention_decode_long_splits(ops, monkeypatch, context, splits):
    """Splits so long that a warp walks more than 32 blocks (it reads the block table 32 blocks at a
    time), an odd and an even number of blocks per warp (it takes them two at a time), and one so
    short that some warps have none.  The plan is forced; pages are scattered."""
    heads, groups, head_dim, page_size = 8, 2, 64, 16
    generator = torch.Generator().manual_seed(context)
    table, positions, token_segment, num_pages = paged_setup([(context, 1)], page_size, generator)
    keys = torch.randn(context + 1, groups, head_dim, generator=generator).to(torch.bfloat16)
    values = torch.randn(context + 1, groups, head_dim, generator=generator).to(torch.bfloat16)
    k_pages = torch.full((num_pages, page_size, groups, head_dim), float("nan"), dtype=torch.bfloat16)
    v_pages = torch.full((num_pages, groups, head_dim, page_size), float("nan"), dtype=torch.bfloat16)
    for position in range(context + 1):
        page = int(table[0, position // page_size])
        k_pages[page, position % page_size] = keys[position]
        v_pages[page, :, :, position % page_size] = values[position]
    blocks_total = (context + 1) // 16 + 1
    per_split = -(-blocks_total // splits)
    monkeypatch.setattr(ops, "decode_attention_plan", lambda *a, **k: (-(-blocks_total // per_split), per_split))
    q = torch.randn(1, heads, head_dim, generator=generator).to(torch.bfloat16)
    out = torch.empty(1, heads * head_dim, dtype=torch.bfloat16, device="cuda")
    flag = status()
    ops.attention_decode(dev(q.reshape(1, -1)), dev(k_pages), dev(v_pages), out, positions=dev(positions), token_segment=dev(token_segment),
                         block_table=dev(table), num_heads=heads, num_groups=groups, head_dim=head_dim, scale=head_dim**-0.5, window=None,
                         max_context=context + 1, status=flag)
    assert flag.item() == 0
    want = reference_attention(q[0].double(), keys.double(), values.double(), context, head_dim**-0.5, None)
    close(out.cpu().reshape(heads, head_dim), want, torch.bfloat16, scale=4.0)


@pytest.mark.parametrize("heads,groups,page_size,window", [
    (4, 1, 16, None), (32, 8, 16, None), (3, 3, 64, None), (6, 2, 16, 33), (24, 8, 32, 300), (8, 1, 16, 5), (16, 1, 48, None), (5, 1, 16, 70),
])
@pytest.mark.parametrize("kind", ["prefill_tcgen05", "prefill_mma", "prefill_tcgen05_split2", "prefill_tcgen05_split5"])
def test_attention_prefill_head_size_64(ops, kind, heads, groups, page_size, window):
    """Both prefill kernels at head size 64 (the tcgen05 one takes no other): 1, 2, 3, 4, 5, 8 and 16 query
    heads per K/V head (128 rows hold 32 tokens of up to 4 heads, fewer tokens of more), windows shorter
    than a tile, pages of one, two, three and four 16-key blocks; rows it must not read hold NaN.  With
    ``_splitN`` every tile that sees at least N tiles of 64 keys is shared by two CTAs that merge their halves
    (contexts of 1 to 32 key tiles here, so some tiles are shared and some are not)."""
    check_attention(ops, kind, torch.bfloat16, heads, groups, 64, page_size, window)


def test_attention_decode_refuses_other_sizes(ops):
    q = torch.zeros(1, 2 * 24, dtype=torch.bfloat16, device="cuda")
    common = dict(positions=torch.zeros(1, dtype=torch.int32, device="cuda"), token_segment=torch.zeros(1, dtype=torch.int32, device="cuda"),
                  block_table=torch.zeros(1, 1, dtype=torch.int32, device="cuda"), num_heads=2, num_groups=1, scale=1.0, window=None, max_context=1, status=status())
    with pytest.raises(ops.KernelError, match="head_dim 24"):
        ops.attention_decode(q, torch.zeros(2, 16, 1, 24, dtype=torch.bfloat16, device="cuda"), torch.zeros(2, 1, 24, 16, dtype=torch.bfloat16, device="cuda"),
                             torch.empty_like(q), head_dim=24, **common)
    q = torch.zeros(1, 2 * 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="page_size 8"):
        ops.attention_decode(q, torch.zeros(2, 8, 1, 32, dtype=torch.bfloat16, device="cuda"), torch.zeros(2, 1, 32, 8, dtype=torch.bfloat16, device="cuda"),
                             torch.empty_like(q), head_dim=32, **common)


def check_attention(ops, kind, dtype, heads, groups, head_dim, page_size, window):
    generator = torch.Generator().manual_seed(head_dim + heads)
    segments = [(0, 40), (300, 1), (page_size * 3 - 1, 2), (255, 3), (700, 5), (2047, 1)]
    table, positions, token_segment, num_pages = paged_setup(segments, page_size, generator)
    tokens = positions.numel()
    k_pages = torch.full((num_pages, page_size, groups, head_dim), float("nan"), dtype=dtype)
    v_pages = torch.full((num_pages, groups, head_dim, page_size), float("nan"), dtype=dtype)  # an unwritten row poisons the result
    history = []
    for row, (context, new) in enumerate(segments):
        length = context + new
        keys = torch.randn(length, groups, head_dim, generator=generator).to(dtype)
        values = torch.randn(length, groups, head_dim, generator=generator).to(dtype)
        first = max(0, context - window + 1) if window else 0  # rows before the first query's window stay unwritten
        for position in range(first, length):
            page = int(table[row, position // page_size])
            k_pages[page, position % page_size] = keys[position]
            v_pages[page, :, :, position % page_size] = values[position]
        history.append((keys.double(), values.double()))
    q = torch.randn(tokens, heads, head_dim, generator=generator).to(dtype)
    out = torch.empty(tokens, heads * head_dim, dtype=dtype, device="cuda")
    flag = status()
    scale = head_dim**-0.5
    call_attention(ops, kind, dev(q.reshape(tokens, -1)), dev(k_pages), dev(v_pages), out, positions, token_segment, table, heads, groups, head_dim, scale, window, flag)
    assert flag.item() == 0
    got = out.cpu().reshape(tokens, heads, head_dim)
    for t in range(tokens):
        keys, values = history[int(token_segment[t])]
        want = reference_attention(q[t].double(), keys, values, int(positions[t]), scale, window)
        # The tensor-core kernels round the probabilities to bfloat16 (2^-9 relative each) before the second
        # product, which moves an output by up to 2^-9 * max|v| (values here reach about 4): four times the
        # absolute tolerance of the plain kernel, whose probabilities stay 32-bit.
        close(got[t], want, dtype, scale=1.0 if kind == "plain" else 4.0)


@pytest.mark.parametrize("kind,dtype", [("plain", torch.float32), ("plain", torch.bfloat16), ("decode", torch.bfloat16), ("prefill", torch.bfloat16)], ids=str)
def test_attention_finds_a_far_key(ops, kind, dtype):
    """One key among a thousand is made to stand out (query and key scaled so its score dominates):
    the output must be that key's value, wherever the key lies: first row, a page's last row, the
    row after a chunk of 256, the query's own position, the window's first row."""
    heads, groups, head_dim, page_size = 2, 1, 32, 16
    length = 1000
    generator = torch.Generator().manual_seed(3)
    table, positions, token_segment, num_pages = paged_setup([(length - 1, 1)], page_size, generator)
    for window, targets in ((None, [0, 15, 16, 255, 256, 511, 998, 999]), (200, [800, 801, 999])):
        for target in targets:
            keys = 0.1 * torch.randn(length, groups, head_dim, generator=generator)
            values = torch.randn(length, groups, head_dim, generator=generator)
            q = 0.1 * torch.randn(1, heads, head_dim, generator=generator)
            keys[target, 0] = 4.0
            q[0, :, :] = 4.0  # score at the target: 16 * 32 / sqrt(32) = 90; elsewhere about 0
            k_pages = torch.zeros(num_pages, page_size, groups, head_dim, dtype=dtype)
            v_pages = torch.zeros(num_pages, groups, head_dim, page_size, dtype=dtype)
            for position in range(length):
                page = int(table[0, position // page_size])
                k_pages[page, position % page_size] = keys[position].to(dtype)
                v_pages[page, :, :, position % page_size] = values[position].to(dtype)
            out = torch.empty(1, heads * head_dim, dtype=dtype, device="cuda")
            call_attention(ops, kind, dev(q.reshape(1, -1).to(dtype)), dev(k_pages), dev(v_pages), out, positions, token_segment, table, heads, groups,
                           head_dim, head_dim**-0.5, window, status())
            want = values[target, 0].to(dtype).double().repeat(heads)
            torch.testing.assert_close(out.cpu().double().flatten(), want, rtol=1e-3, atol=1e-3, msg=f"window {window}, key {target}")


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("dim,taps,bias", [(64, 3, False), (96, 4, True), (200, 2, True), (130, 7, False), (48, 1, True)])
def test_short_conv(ops, dtype, dim, taps, bias):
    """Ragged portions, some shorter than the state, over several steps: state carried in slots."""
    generator = torch.Generator().manual_seed(dim + taps)
    history = max(taps - 1, 1)
    slots = 5
    state = torch.full((slots, history, dim), 7.0, dtype=dtype, device="cuda")
    state[[4, 1, 2]] = 0  # the requests' slots start at zero; slots 0 and 3 must stay untouched
    weight = torch.randn(dim, taps, generator=generator)
    conv_bias = torch.randn(dim, generator=generator) if bias else None
    lengths = {4: [5, 1, 2, 1, 9], 1: [1, 1, 1, 3, 2], 2: [12, 2, 1, 1, 1]}  # per slot, per step
    inputs = {slot: torch.randn(sum(sizes), 3 * dim, generator=generator).to(dtype) for slot, sizes in lengths.items()}
    done = {slot: 0 for slot in lengths}

    def whole(proj: torch.Tensor) -> torch.Tensor:
        pre, post, x = proj[:, :dim].double(), proj[:, dim : 2 * dim].double(), proj[:, 2 * dim :].double()
        u = rnd(pre * x, dtype)
        padded = torch.cat([torch.zeros(taps - 1, dim, dtype=torch.float64), u])
        conv = sum(padded[k : k + proj.shape[0]] * weight[:, k].double() for k in range(taps))
        if conv_bias is not None:
            conv = conv + conv_bias.double()
        return post * rnd(conv, dtype)

    expected = {slot: whole(proj) for slot, proj in inputs.items()}
    for step in range(5):
        order = [4, 1, 2] if step % 2 == 0 else [2, 4, 1]
        sizes = [lengths[slot][step] for slot in order]
        proj = torch.cat([inputs[slot][done[slot] : done[slot] + size] for slot, size in zip(order, sizes)])
        starts = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int32)
        token_segment = torch.repeat_interleave(torch.arange(3, dtype=torch.int32), torch.tensor(sizes))
        out = torch.empty(sum(sizes), dim, dtype=dtype, device="cuda")
        flag = status()
        ops.short_conv(
            dev(proj), state if taps > 1 else state[:, :0], dev(weight), None if conv_bias is None else dev(conv_bias), out,
            token_segment=dev(token_segment), segment_start=dev(torch.from_numpy(starts)), segment_length=dev(torch.tensor(sizes, dtype=torch.int32)),
            segment_slot=dev(torch.tensor(order, dtype=torch.int32)), segments=3, status=flag)
        assert flag.item() == 0
        host = out.cpu()
        for slot, size, start in zip(order, sizes, starts):
            close(host[start : start + size], expected[slot][done[slot] : done[slot] + size], dtype, scale=4)
            done[slot] += size
    assert (state[[0, 3]] == 7.0).all()
    if taps > 1:  # the state is the last taps-1 gated inputs
        for slot, proj in inputs.items():
            u = rnd(proj[:, :dim].double() * proj[:, 2 * dim :].double(), dtype)
            close(state[slot].cpu(), u[-(taps - 1) :], dtype, scale=4)


@pytest.mark.parametrize("taps,bias", [(2, False), (3, True), (4, False)])
def test_short_conv_many_tokens(ops, taps, bias):
    """Hundreds of tokens in a step: long portions beside portions shorter than the history, each
    continuing the state that an earlier step left (two steps); the channel count is no power of two."""
    dtype, dim, slots = torch.bfloat16, 136, 6
    generator = torch.Generator().manual_seed(taps)
    history = taps - 1
    state = torch.zeros((slots, history, dim), dtype=dtype, device="cuda")
    weight = torch.randn(dim, taps, generator=generator)
    conv_bias = torch.randn(dim, generator=generator) if bias else None
    lengths = {0: [131, 70], 5: [1, 3], 2: [2, 1], 3: [157, 200], 1: [66, 9]}  # per slot, per step
    inputs = {slot: torch.randn(sum(sizes), 3 * dim, generator=generator).to(dtype) for slot, sizes in lengths.items()}

    def whole(proj: torch.Tensor) -> torch.Tensor:
        pre, post, x = proj[:, :dim].double(), proj[:, dim : 2 * dim].double(), proj[:, 2 * dim :].double()
        u = rnd(pre * x, dtype)
        padded = torch.cat([torch.zeros(taps - 1, dim, dtype=torch.float64), u])
        conv = sum(padded[k : k + proj.shape[0]] * weight[:, k].double() for k in range(taps))
        if conv_bias is not None:
            conv = conv + conv_bias.double()
        return post * rnd(conv, dtype)

    expected = {slot: whole(proj) for slot, proj in inputs.items()}
    done = {slot: 0 for slot in lengths}
    for step in range(2):
        order = list(lengths) if step == 0 else list(lengths)[::-1]
        sizes = [lengths[slot][step] for slot in order]
        assert sum(sizes) >= 256
        proj = torch.cat([inputs[slot][done[slot] : done[slot] + size] for slot, size in zip(order, sizes)])
        starts = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int32)
        token_segment = torch.repeat_interleave(torch.arange(len(order), dtype=torch.int32), torch.tensor(sizes))
        out = torch.empty(sum(sizes), dim, dtype=dtype, device="cuda")
        flag = status()
        ops.short_conv(
            dev(proj), state, dev(weight), None if conv_bias is None else dev(conv_bias), out,
            token_segment=dev(token_segment), segment_start=dev(torch.from_numpy(starts)), segment_length=dev(torch.tensor(sizes, dtype=torch.int32)),
            segment_slot=dev(torch.tensor(order, dtype=torch.int32)), segments=len(order), status=flag)
        assert flag.item() == 0
        host = out.cpu()
        for slot, size, start in zip(order, sizes, starts):
            close(host[start : start + size], expected[slot][done[slot] : done[slot] + size], dtype, scale=4)
            done[slot] += size
    for slot, proj in inputs.items():
        u = rnd(proj[:, :dim].double() * proj[:, 2 * dim :].double(), dtype)
        close(state[slot].cpu(), u[-history:], dtype, scale=4)



@pytest.mark.parametrize("dim,taps,bias,slices", [(136, 3, True, 3), (1024, 3, False, 4), (64, 1, True, 2), (200, 4, True, 0), (96, 2, False, 5)])
def test_short_conv_of_single_tokens_in_one_kernel(ops, dim, taps, bias, slices):
    """A step in which every portion is one token: the slices' sum (``slices`` > 0: the in-projection comes as partial
    sums), the convolution and the state update in one kernel.  Three steps over requests in scrambled slots, bit for
    bit against the kernels for general steps (run on a copy of the state), and the state against the inputs."""
    from ctypes import c_int

    dtype, slots, tokens = torch.bfloat16, 50, 40
    generator = torch.Generator().manual_seed(dim + taps)
    history = taps - 1
    weight = torch.randn(dim, taps, generator=generator)
    conv_bias = torch.randn(dim, generator=generator) if bias else None
    state = (torch.randn(slots, history, dim, generator=generator)).to(dtype).cuda()
    reference_state = state.clone()
    order = torch.randperm(slots, generator=generator)[:tokens].to(torch.int32)
    token_segment = torch.arange(tokens, dtype=torch.int32)
    starts, lengths = torch.arange(tokens, dtype=torch.int32), torch.ones(tokens, dtype=torch.int32)
    device_weight, device_bias = dev(weight), None if conv_bias is None else dev(conv_bias)   # held: the direct call below takes raw pointers
    inputs = []
    for step in range(3):
        if slices:
            partials = torch.randn(slices, tokens, 3 * dim, generator=generator).cuda()
            total = torch.zeros(tokens, 3 * dim, device="cuda")
            for s in range(slices):
                total += partials[s]
            proj = total.to(dtype)
            given = ops.SlicedSum(partials, dtype)
        else:
            proj = torch.randn(tokens, 3 * dim, generator=generator).to(dtype).cuda()
            given = proj
        inputs.append(proj.cpu())
        out, expected = torch.empty(tokens, dim, dtype=dtype, device="cuda"), torch.empty(tokens, dim, dtype=dtype, device="cuda")
        flag = status()
        lists = dict(token_segment=dev(token_segment), segment_start=dev(starts), segment_length=dev(lengths), segment_slot=dev(order))
        before = ops.launch_count()
        ops.short_conv(given, state if taps > 1 else state[:, :0], device_weight, device_bias, out, segments=tokens, status=flag, **lists)
        assert ops.launch_count() - before == 1 and flag.item() == 0
        # the kernels for general steps, called directly on the summed in-projection
        code = ops._lib().lb_short_conv(
            ops._ptr(proj), ops._ptr(reference_state), ops._ptr(device_weight), ops._ptr(device_bias), ops._ptr(expected),
            ops._ptr(lists["token_segment"]), ops._ptr(lists["segment_start"]), ops._ptr(lists["segment_length"]), ops._ptr(lists["segment_slot"]),
            c_int(tokens), c_int(tokens), c_int(dim), c_int(taps), c_int(slots), c_int(ops.dtype_code(dtype)), ops._ptr(flag), ops._stream())
        assert code == 0
        torch.cuda.synchronize()
        assert torch.equal(out, expected)
        assert torch.equal(state, reference_state)
    if taps > 1:
        host = state.cpu()
        for place, slot in enumerate(order.tolist()):
            u = [rnd(proj[place, :dim].double() * proj[place, 2 * dim :].double(), dtype) for proj in inputs]
            close(host[slot, -1], u[-1], dtype)
            if history >= 2:
                close(host[slot, -2], u[-2], dtype)
        untouched = torch.ones(slots, dtype=torch.bool)
        untouched[order.long()] = False
        assert untouched.any()


# ----------------------------------------------------------------------- weight-streaming products
SKINNY_SHAPES = [(1, 64, 16), (5, 96, 40), (8, 2048, 2048), (9, 2080, 176), (16, 4096, 8192), (3, 32, 65536)]


@pytest.mark.parametrize("tokens,width,rows", SKINNY_SHAPES)
def test_skinny_linear_store_and_float(ops, tokens, width, rows):
    generator = torch.Generator().manual_seed(tokens * width)
    x = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    w = (torch.randn(rows, width, generator=generator) / math.sqrt(width)).to(torch.bfloat16)
    assert ops.skinny_supported(dev(x), rows)
    want = x.double() @ w.double().T
    close(ops.linear(dev(x), dev(w)), want, torch.bfloat16)
    got = ops.linear(dev(x), dev(w), out_dtype=torch.float32)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-5)


def test_linear_falls_back_to_the_library_for_other_sizes(ops):
    generator = torch.Generator().manual_seed(0)
    for tokens, width, rows, dtype in ((17, 64, 32, torch.bfloat16), (4, 40, 32, torch.bfloat16), (4, 64, 20, torch.bfloat16), (4, 64, 32, torch.float32)):
        x = torch.randn(tokens, width, generator=generator).to(dtype)
        w = torch.randn(rows, width, generator=generator).to(dtype)
        assert not ops.skinny_supported(dev(x), rows)
        close(ops.linear(dev(x), dev(w)), x.double() @ w.double().T, dtype, scale=8)


@pytest.mark.parametrize("tokens,width,rows", SKINNY_SHAPES[:5])
def test_skinny_residual_add_and_gated(ops, tokens, width, rows):
    generator = torch.Generator().manual_seed(tokens + rows)
    x = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    w = (torch.randn(rows, width, generator=generator) / math.sqrt(width)).to(torch.bfloat16)
    residual = torch.randn(tokens, rows, generator=generator)
    on_device = dev(residual.clone())
    assert ops.linear_accumulate(dev(x), dev(w), on_device) is None
    want = residual.double() + rnd(x.double() @ w.double().T, torch.bfloat16)
    torch.testing.assert_close(on_device.cpu().double(), want, rtol=1e-5, atol=2e-2)
    torch.testing.assert_close(on_device.cpu().double(), residual.double() + x.double() @ w.double().T, rtol=1e-2, atol=2e-2)
    # gated: rows [0, hidden) are "up", rows [hidden, 2 hidden) are "gate"
    up_gate = (torch.randn(2 * rows, width, generator=generator) / math.sqrt(width)).to(torch.bfloat16)
    got = ops.gated_linear(dev(x), dev(up_gate), "silu")
    fused = x.double() @ up_gate.double().T
    up, gate = rnd(fused[:, :rows], torch.bfloat16), rnd(fused[:, rows:], torch.bfloat16)
    close(got, up * rnd(gate * torch.sigmoid(gate), torch.bfloat16), torch.bfloat16, scale=2)


@pytest.mark.parametrize("dim,width,taps,bias", [(64, 64, 3, False), (96, 160, 4, True), (2048, 2048, 3, False), (48, 32, 1, True), (80, 96, 6, True)])
def test_skinny_short_conv(ops, dim, width, taps, bias):
    """The fused in-projection + convolution equals the plain formula over whole sequences, for
    ragged portions (some shorter than the state) over several steps."""
    dtype = torch.bfloat16
    generator = torch.Generator().manual_seed(dim + taps)
    history = max(taps - 1, 1)
    state = torch.full((5, history, dim), 7.0, dtype=dtype, device="cuda")
    state[[4, 1, 2]] = 0
    in_proj = (torch.randn(3 * dim, width, generator=generator) / math.sqrt(width)).to(dtype)
    weight = torch.randn(dim, taps, generator=generator)
    conv_bias = torch.randn(dim, generator=generator) if bias else None
    lengths = {4: [5, 1, 2, 1, 6], 1: [1, 1, 1, 3, 2], 2: [7, 2, 1, 1, 1]}
    inputs = {slot: torch.randn(sum(sizes), width, generator=generator).to(dtype) for slot, sizes in lengths.items()}

    def whole(x: torch.Tensor) -> torch.Tensor:
        proj = rnd(x.double() @ in_proj.double().T, dtype)
        pre, post, gated = proj[:, :dim], proj[:, dim : 2 * dim], proj[:, 2 * dim :]
        u = rnd(pre * gated, dtype)
        padded = torch.cat([torch.zeros(taps - 1, dim, dtype=torch.float64), u])
        conv = sum(padded[k : k + x.shape[0]] * weight[:, k].double() for k in range(taps))
        if conv_bias is not None:
            conv = conv + conv_bias.double()
        return post * rnd(conv, dtype), u

    expected = {slot: whole(x) for slot, x in inputs.items()}
    done = {slot: 0 for slot in lengths}
    for step in range(5):
        order = [4, 1, 2] if step % 2 == 0 else [2, 4, 1]
        sizes = [lengths[slot][step] for slot in order]
        x = torch.cat([inputs[slot][done[slot] : done[slot] + size] for slot, size in zip(order, sizes)])
        starts = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int32)
        token_segment = torch.repeat_interleave(torch.arange(3, dtype=torch.int32), torch.tensor(sizes))
        flag = status()
        assert ops.skinny_supported(dev(x), dim)
        out = ops.short_conv_linear(
            dev(x), dev(in_proj), state if taps > 1 else state[:, :0], dev(weight), None if conv_bias is None else dev(conv_bias),
            token_segment=dev(token_segment), segment_start=dev(torch.from_numpy(starts)), segment_length=dev(torch.tensor(sizes, dtype=torch.int32)),
            segment_slot=dev(torch.tensor(order, dtype=torch.int32)), segments=3, status=flag)
        assert flag.item() == 0
        host = out.cpu()
        for slot, size, start in zip(order, sizes, starts):
            close(host[start : start + size], expected[slot][0][done[slot] : done[slot] + size], dtype, scale=4)
            done[slot] += size
    assert (state[[0, 3]] == 7.0).all()
    if taps > 1:
        for slot in lengths:
            close(state[slot].cpu(), expected[slot][1][-(taps - 1) :], dtype, scale=4)


# ------------------------------------------------------------------------------- tcgen05 products
TC_SHAPES = [(17, 64, 128), (33, 2048, 2048), (64, 2080, 1000), (100, 512, 6144), (256, 8192, 256), (300, 96, 136), (2048, 2048, 384), (1, 64, 8), (2100, 328, 2600), (129, 72, 120), (300, 96, 134)]


@pytest.mark.parametrize("tokens,width,rows", TC_SHAPES)
def test_tcgen05_linear(ops, tokens, width, rows):
    """Tile edges in every direction (rows no multiple of 128, tokens no multiple of the tile, widths
    no multiple of 64), one K slice and several, all three epilogues; above 128 tokens with one slice
    the walking kernel with 256-token tiles runs, in one shape with more tiles than the GPU has SMs,
    and in one whose output rows are not 16-byte aligned, so that it cannot leave by bulk stores."""
    generator = torch.Generator().manual_seed(tokens + width)
    x = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    w = (torch.randn(rows, width, generator=generator) / math.sqrt(width)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    for slices in (1, 3):
        got = ops.linear_tcgen05(dev(x), dev(w), "store_float", slices=slices)
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-4, msg=lambda m: f"float32 store, {slices} slices: {m}")
        close(ops.linear_tcgen05(dev(x), dev(w), "store", slices=slices), want, torch.bfloat16)
        residual = torch.randn(tokens, rows, generator=generator)
        on_device = dev(residual.clone())
        ops.linear_tcgen05(dev(x), dev(w), "residual_add", residual=on_device, slices=slices)
        torch.testing.assert_close(on_device.cpu().double(), residual.double() + rnd(want, torch.bfloat16), rtol=1e-5, atol=2e-2)
    again = ops.linear_tcgen05(dev(x), dev(w), "store_float", slices=3)
    assert torch.equal(again, ops.linear_tcgen05(dev(x), dev(w), "store_float", slices=3))  # slices are summed in order: same bits


@pytest.mark.parametrize("tokens,width,hidden,activation", [(20, 64, 64, "silu"), (100, 2048, 1000, "silu"), (300, 160, 200, "gelu"), (2048, 512, 1024, "silu"), (2100, 328, 1400, "silu"), (260, 64, 100, "silu")])
def test_tcgen05_gated(ops, tokens, width, hidden, activation):
    generator = torch.Generator().manual_seed(tokens + hidden)
    x = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    up_gate = (torch.randn(2 * hidden, width, generator=generator) / math.sqrt(width)).to(torch.bfloat16)
    fused = x.double() @ up_gate.double().T
    up, gate = rnd(fused[:, :hidden], torch.bfloat16), rnd(fused[:, hidden:], torch.bfloat16)
    act = gate * torch.sigmoid(gate) if activation == "silu" else 0.5 * gate * (1 + torch.erf(gate / math.sqrt(2)))
    got = ops.linear_tcgen05(dev(x), dev(up_gate), "gated", activation=activation)
    assert got.shape == (tokens, hidden)
    close(got, up * rnd(act, torch.bfloat16), torch.bfloat16, scale=2)


@pytest.mark.parametrize("tile", ["64", "128", "256", "512"])
@pytest.mark.parametrize("tokens,width,rows", [(300, 200, 384), (1000, 2048, 640), (2100, 328, 2600), (513, 72, 130)])
def test_tcgen05_walking_tiles(ops, monkeypatch, tile, tokens, width, rows):
    """Every tile shape of the walking kernel forced in turn (64, 128 or 256 tokens, and "512": a
    pair of CTAs on 256 rows x 256 tokens), on sizes whose edges fall inside tiles in every direction:
    an odd number of 128-row tiles leaves the pair's second CTA with rows beyond the matrix."""
    monkeypatch.setenv("LALAMO_B200_TCGEN05_TILE", tile)
    generator = torch.Generator().manual_seed(tokens + rows)
    x = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    w = (torch.randn(rows, width, generator=generator) / math.sqrt(width)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    got = ops.linear_tcgen05(dev(x), dev(w), "store_float", slices=1)
    torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-4)
    close(ops.linear_tcgen05(dev(x), dev(w), "store", slices=1), want, torch.bfloat16)
    if tile != "64":
        # the walkers' items as (tile, K slice) pairs: partial sums through 3-D bulk stores (or plain stores where the
        # rows are not 16-byte aligned), the last slice shorter than the others, summed by the consumer
        sliced = ops.linear_tcgen05(dev(x), dev(w), "residual_add", residual=dev(torch.zeros(tokens, rows)), slices=3, defer_sum=True)
        assert isinstance(sliced, ops.SlicedSum) and sliced.partials.shape[0] == ops._settled_slices(3, width)
        torch.testing.assert_close(sliced.partials.double().sum(0).cpu(), want, rtol=1e-4, atol=1e-4)
    residual = torch.randn(tokens, rows, generator=generator)
    on_device = dev(residual.clone())
    ops.linear_tcgen05(dev(x), dev(w), "residual_add", residual=on_device, slices=1)
    torch.testing.assert_close(on_device.cpu().double(), residual.double() + rnd(want, torch.bfloat16), rtol=1e-5, atol=2e-2)
    hidden = rows // 2
    fused = want
    up, gate = rnd(fused[:, :hidden], torch.bfloat16), rnd(fused[:, hidden:], torch.bfloat16)
    gated = ops.linear_tcgen05(dev(x), dev(w), "gated", activation="silu")
    close(gated, up * rnd(gate * torch.sigmoid(gate), torch.bfloat16), torch.bfloat16, scale=2)


def test_tcgen05_refuses_unaligned_rows(ops):
    x = torch.zeros(20, 36, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.linear_tcgen05(x, torch.zeros(8, 36, dtype=torch.bfloat16, device="cuda"))
    assert not ops.tcgen05_supported(x, 8)
