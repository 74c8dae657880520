"""The decode-attention entry point that allocates nothing (its scratch is a device
array inside the library), called the way its users call it: through the exported C
symbol of the shared library, with raw pointers. Collected last on purpose (the file
name sorts after every other test file), so that a run that stops at the first
failure has already run everything else. It must pass alone in a fresh process and
after the other tests."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_the_regular_one():
    from semantic_aware_adaptive_kv_cache_precision_b200 import ops
    from semantic_aware_adaptive_kv_cache_precision_b200.csrc import build
    from semantic_aware_adaptive_kv_cache_precision_b200.ops.attention import tensor_map

    lib = ctypes.CDLL(str(build.build("attention_decode")))
    entry = lib.sakv_decode_attention_static_scratch
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    entry.argtypes = [P, P, P, L, P, P, I, P, I, I, I, I, I, F, I, ctypes.c_char_p, I, P]
    entry.restype = I

    rng = np.random.default_rng(0)
    heads, kv_heads, d, splits = 12, 2, 128, 4
    lengths = [700, 65, 2048, 1]
    blocks = 64
    k_cache = torch.as_tensor(rng.standard_normal((blocks, kv_heads, 64, d))).to("cuda").to(
        torch.bfloat16).contiguous()
    v_cache = torch.as_tensor(rng.standard_normal((blocks, kv_heads, 64, d))).to("cuda").to(
        torch.bfloat16).contiguous()
    order = rng.permutation(blocks)
    table = np.full((len(lengths), 32), -1, dtype=np.int32)
    at = 0
    for i, n in enumerate(lengths):
        for b in range(-(-n // 64)):
            table[i, b] = order[at]
            at += 1
    table_d = torch.as_tensor(table).to("cuda")
    lens_d = torch.as_tensor(lengths, dtype=torch.int32).to("cuda")
    scale = d ** -0.5
    stream = torch.cuda.current_stream().cuda_stream
    why = ctypes.create_string_buffer(256)

    for call in range(2):                      # twice in a row: the scratch is shared and kept
        qkv = torch.as_tensor(rng.standard_normal((len(lengths), (heads + 2 * kv_heads) * d))).to(
            "cuda").to(torch.bfloat16).contiguous()
        want = ops.attention_decode(qkv, k_cache, v_cache, lens_d, table_d, heads, kv_heads, d,
                                    scale, None, max(lengths), splits=splits)
        got = torch.full_like(want, float("nan"))
        code = entry(tensor_map(k_cache), tensor_map(v_cache), qkv.data_ptr(), qkv.stride(0),
                     lens_d.data_ptr(), table_d.data_ptr(), table_d.shape[1], got.data_ptr(),
                     len(lengths), heads, kv_heads, d, splits, scale, 0, why, len(why), stream)
        assert code == 0, why.value.decode()
        torch.cuda.synchronize()
        # the same kernels in the same order: the same bits as the entry point that takes
        # its scratch from the caller
        assert torch.equal(got, want), f"call {call}: differs from the regular entry point"
        # and the right answer: each query against a float64 softmax over its sequence's keys,
        # within the bf16 rounding of the probabilities and of the result
        q = qkv[:, :heads * d].float().cpu().numpy().astype(np.float64).reshape(-1, heads, d)
        keys = k_cache.float().cpu().numpy().astype(np.float64)
        values = v_cache.float().cpu().numpy().astype(np.float64)
        for i, n in enumerate(lengths):
            mine = table[i, :-(-n // 64)]
            k = keys[mine].transpose(0, 2, 1, 3).reshape(-1, kv_heads, d)[:n]
            v = values[mine].transpose(0, 2, 1, 3).reshape(-1, kv_heads, d)[:n]
            for h in range(heads):
                g = h // (heads // kv_heads)
                s = (k[:, g] @ q[i, h]) * scale
                p = np.exp(s - s.max())
                ref = (p / p.sum()) @ v[:, g]
                np.testing.assert_allclose(got[i, h * d:(h + 1) * d].float().cpu().numpy(), ref,
                                           rtol=0, atol=1.5e-2,
                                           err_msg=f"call {call}, sequence {i}, head {h}")

    # a problem larger than the built-in scratch is refused, with a sentence, before any launch
    before = got.clone()
    code = entry(tensor_map(k_cache), tensor_map(v_cache), qkv.data_ptr(), qkv.stride(0),
                 lens_d.data_ptr(), table_d.data_ptr(), table_d.shape[1], got.data_ptr(),
                 60000, heads, kv_heads, d, 32, scale, 0, why, len(why), stream)
    assert code == 1 and b"built-in scratch holds 2097152" in why.value
    torch.cuda.synchronize()
    assert torch.equal(before, got)
