"""The attention entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library cannot hand it scratch memory, because they run where calling an
allocator is not allowed (while someone else's stream capture is going on, on a thread that must not
take allocator or driver locks, inside a host program that gave them no memory budget).  For them
``lb_attention_decode_static`` keeps its scratch in a fixed array inside the library.  This test calls
it several times in a row with cases of different sizes (so that each call finds another call's partial
results in the array) and compares every call with a float64 attention over the same keys and values,
then with the allocating entry point, whose bits it must reproduce; it also checks the refusal of sizes
beyond the built-in maximum.  The file sorts last so that a run that stops at the first failure has
run everything else before.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def build_case(seed: int, tokens: int, heads: int, groups: int, head_dim: int, page_size: int = 16, longest: int = 700):
    """Random queries, and keys and values scattered over pages; rows of the pool that belong to no
    request hold NaN.  Returns the device tensors and the dense keys and values of every request."""
    generator = torch.Generator().manual_seed(seed)
    contexts = torch.randint(1, longest, (tokens,), generator=generator).tolist()
    blocks = [-(-(context + 1) // page_size) for context in contexts]
    num_pages = sum(blocks) + 2
    order = torch.randperm(num_pages, generator=generator).tolist()
    table = torch.full((tokens, max(blocks)), -1, dtype=torch.int32)
    k_pages = torch.full((num_pages, page_size, groups, head_dim), float("nan"), dtype=torch.bfloat16)
    v_pages = torch.full((num_pages, groups, head_dim, page_size), float("nan"), dtype=torch.bfloat16)
    dense = []
    cursor = 0
    for row, count in enumerate(blocks):
        pages = order[cursor : cursor + count]
        table[row, :count] = torch.tensor(pages, dtype=torch.int32)
        cursor += count
        keys = torch.randn(contexts[row] + 1, groups, head_dim, generator=generator).to(torch.bfloat16)
        values = torch.randn(contexts[row] + 1, groups, head_dim, generator=generator).to(torch.bfloat16)
        for position in range(contexts[row] + 1):
            k_pages[pages[position // page_size], position % page_size] = keys[position]
            v_pages[pages[position // page_size], :, :, position % page_size] = values[position]
        dense.append((keys.double(), values.double()))
    queries = torch.randn(tokens, heads, head_dim, generator=generator).to(torch.bfloat16)
    case = {
        "q": queries.reshape(tokens, heads * head_dim).cuda(),
        "k": k_pages.cuda(),
        "v": v_pages.cuda(),
        "positions": torch.tensor(contexts, dtype=torch.int32).cuda(),
        "segments": torch.arange(tokens, dtype=torch.int32).cuda(),
        "table": table.cuda(),
        "status": torch.zeros(1, dtype=torch.int32).cuda(),
        "queries": queries.double(),
        "dense": dense,
        "contexts": contexts,
    }
    return case, num_pages, max(contexts) + 1


def call_static(library, case, tokens, heads, groups, head_dim, num_pages, splits, blocks_per_split, page_size=16, window=0, token_list=None, fill=0.0):
    out = torch.full((case["q"].shape[0], heads * head_dim), fill, dtype=torch.bfloat16, device="cuda")
    message = ctypes.create_string_buffer(512)
    function = library.lb_attention_decode_static
    function.restype = c_int
    code = function(
        c_void_p(case["q"].data_ptr()), c_void_p(case["k"].data_ptr()), c_void_p(case["v"].data_ptr()), c_void_p(out.data_ptr()),
        c_void_p(case["positions"].data_ptr()), c_void_p(case["segments"].data_ptr()), c_void_p(case["table"].data_ptr()),
        c_void_p(token_list.data_ptr() if token_list is not None else 0),
        c_int(tokens), c_int(heads), c_int(groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(case["table"].shape[1]),
        c_float(head_dim**-0.5), c_int(window), c_int(splits), c_int(blocks_per_split), c_void_p(case["status"].data_ptr()),
        c_void_p(torch.cuda.current_stream().cuda_stream), message, c_int(512))
    return code, out, message.value.decode()


def expected_rows(case, heads, head_dim, window):
    """The float64 attention of every token, from the dense keys and values."""
    from test_kernels_gpu import reference_attention

    rows = [reference_attention(case["queries"][token], *case["dense"][token], case["contexts"][token], head_dim**-0.5, window or None)
            for token in range(len(case["contexts"]))]
    return torch.stack(rows).reshape(len(rows), heads * head_dim)


# Each case runs after another one of other sizes: the array still holds that call's partial results, laid
# out for other token, head and split counts, so that a slot the kernels read without having written it
# shows.  The second case is smaller than the first (it leaves most of what the first wrote in place), the
# third has a ring of keys and values beyond 48 KB (head size 128), the fourth runs a listed subset of its
# tokens under a window.
CASES = [
    dict(tokens=9, heads=8, groups=2, head_dim=64, window=0, listed=False),
    dict(tokens=3, heads=6, groups=3, head_dim=32, window=0, listed=False),
    dict(tokens=5, heads=8, groups=2, head_dim=128, window=0, listed=False),
    dict(tokens=7, heads=4, groups=1, head_dim=64, window=100, listed=True),
]


def test_static_scratch_entry_point_matches_the_float64_attention_call_after_call():
    from lalamo_b200 import native, ops

    library = native.library()
    for seed, shape in enumerate(CASES):
        tokens, heads, groups, head_dim, window = (shape[name] for name in ("tokens", "heads", "groups", "head_dim", "window"))
        case, num_pages, max_context = build_case(seed, tokens, heads, groups, head_dim)
        want = expected_rows(case, heads, head_dim, window)
        listed = torch.arange(tokens - 1, -1, -2, dtype=torch.int32).cuda() if shape["listed"] else None
        running = tokens if listed is None else listed.numel()
        splits, blocks_per_split = ops.decode_attention_plan(running, heads, groups, max_context, window or None, head_dim)
        code, out, message = call_static(library, case, running, heads, groups, head_dim, num_pages, splits, blocks_per_split, window=window,
                                         token_list=listed, fill=123.0)
        assert code == 0, message
        rows = torch.arange(tokens) if listed is None else listed.cpu().long()
        torch.testing.assert_close(out.cpu().double()[rows], want[rows], rtol=2e-2, atol=4e-3)
        if listed is not None:
            others = torch.ones(tokens, dtype=torch.bool)
            others[rows] = False
            assert (out.cpu()[others] == 123.0).all()  # tokens that are not listed are left alone
        # the allocating entry point gives the same bits: the two share their kernels
        same = torch.full_like(out, 123.0)
        ops.attention_decode(case["q"], case["k"], case["v"], same, positions=case["positions"], token_segment=case["segments"],
                             block_table=case["table"], num_heads=heads, num_groups=groups, head_dim=head_dim, scale=head_dim**-0.5,
                             window=window or None, max_context=max_context, status=case["status"], token_list=listed,
                             num_listed=None if listed is None else listed.numel())
        assert torch.equal(out, same)
        assert case["status"].item() == 0


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from lalamo_b200 import native

    library = native.library()
    tokens, heads, groups, head_dim = 64, 32, 8, 128
    case, num_pages, _ = build_case(7, tokens, heads, groups, head_dim, longest=40)
    code, _, message = call_static(library, case, tokens, heads, groups, head_dim, num_pages, splits=64, blocks_per_split=1)
    assert code == -4 and "exceed the built-in 4194304" in message  # 64 * 32 * 64 * 130 floats
    code, _, message = call_static(library, case, tokens, heads, groups, 24, num_pages, splits=1, blocks_per_split=64)
    assert code == -2 and "head_dim" in message
