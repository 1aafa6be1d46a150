"""The attention entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library cannot hand it scratch memory, because they run where calling an
allocator is not allowed (while someone else's stream capture is going on, on a thread that must not
take allocator or driver locks, inside a host program that gave them no memory budget).  For them
``lb_attention_decode_static`` keeps its scratch in a fixed array inside the library.  This test calls
it twice in a row and compares with the allocating entry point; it also checks the refusal of sizes
beyond the built-in maximum.  The file sorts last so that a run that stops at the first failure has
run everything else before.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def build_case(seed: int, tokens: int, heads: int, groups: int, head_dim: int, page_size: int = 16):
    generator = torch.Generator().manual_seed(seed)
    contexts = torch.randint(1, 700, (tokens,), generator=generator).tolist()
    blocks = [-(-(context + 1) // page_size) for context in contexts]
    num_pages = sum(blocks) + 2
    order = torch.randperm(num_pages, generator=generator).tolist()
    table = torch.full((tokens, max(blocks)), -1, dtype=torch.int32)
    cursor = 0
    for row, count in enumerate(blocks):
        table[row, :count] = torch.tensor(order[cursor : cursor + count], dtype=torch.int32)
        cursor += count
    case = {
        "q": torch.randn(tokens, heads * head_dim, generator=generator).to(torch.bfloat16).cuda(),
        "k": torch.randn(num_pages, page_size, groups, head_dim, generator=generator).to(torch.bfloat16).cuda(),
        "v": torch.randn(num_pages, groups, head_dim, page_size, generator=generator).to(torch.bfloat16).cuda(),
        "positions": torch.tensor(contexts, dtype=torch.int32).cuda(),
        "segments": torch.arange(tokens, dtype=torch.int32).cuda(),
        "table": table.cuda(),
        "status": torch.zeros(1, dtype=torch.int32).cuda(),
    }
    return case, num_pages, max(contexts) + 1


def call_static(library, case, tokens, heads, groups, head_dim, num_pages, splits, blocks_per_split, page_size=16):
    out = torch.empty(tokens, heads * head_dim, dtype=torch.bfloat16, device="cuda")
    message = ctypes.create_string_buffer(512)
    function = library.lb_attention_decode_static
    function.restype = c_int
    code = function(
        c_void_p(case["q"].data_ptr()), c_void_p(case["k"].data_ptr()), c_void_p(case["v"].data_ptr()), c_void_p(out.data_ptr()),
        c_void_p(case["positions"].data_ptr()), c_void_p(case["segments"].data_ptr()), c_void_p(case["table"].data_ptr()), c_void_p(0),
        c_int(tokens), c_int(heads), c_int(groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(case["table"].shape[1]),
        c_float(head_dim**-0.5), c_int(0), c_int(splits), c_int(blocks_per_split), c_void_p(case["status"].data_ptr()),
        c_void_p(torch.cuda.current_stream().cuda_stream), message, c_int(512))
    return code, out, message.value.decode()


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from lalamo_b200 import native, ops

    library = native.library()
    for seed, (tokens, heads, groups, head_dim) in enumerate([(5, 8, 2, 64), (9, 6, 3, 32)]):
        case, num_pages, max_context = build_case(seed, tokens, heads, groups, head_dim)
        expected = torch.empty(tokens, heads * head_dim, dtype=torch.bfloat16, device="cuda")
        ops.attention_decode(case["q"], case["k"], case["v"], expected, positions=case["positions"], token_segment=case["segments"],
                             block_table=case["table"], num_heads=heads, num_groups=groups, head_dim=head_dim, scale=head_dim**-0.5,
                             window=None, max_context=max_context, status=case["status"])
        splits, blocks_per_split = ops.decode_attention_plan(tokens, heads, groups, max_context, None)
        for _ in range(2):  # the second call finds the array as the first one left it
            code, out, message = call_static(library, case, tokens, heads, groups, head_dim, num_pages, splits, blocks_per_split)
            assert code == 0, message
            torch.testing.assert_close(out.float(), expected.float(), rtol=2e-2, atol=2e-3)
        assert case["status"].item() == 0


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from lalamo_b200 import native

    library = native.library()
    tokens, heads, groups, head_dim = 64, 32, 8, 128
    case, num_pages, _ = build_case(7, tokens, heads, groups, head_dim)
    code, _, message = call_static(library, case, tokens, heads, groups, head_dim, num_pages, splits=64, blocks_per_split=1)
    assert code == -4 and "exceed the built-in 4194304" in message  # 64 * 32 * 64 * 130 floats
    code, _, message = call_static(library, case, tokens, heads, groups, 24, num_pages, splits=1, blocks_per_split=64)
    assert code == -2 and "head_dim" in message
