"""The allocation-free entry point of the decode attention kernel
(rllm_attention_decode_bf16_static, declared in
rllm_b200/kernels/csrc/attention_decode_static.h), called the way a host
without an allocator would call it: through its exported C symbol, with raw
pointers.  Some callers of this library cannot allocate device memory when they
call it - a plain C host without PyTorch's allocator, a process whose pool
already owns all of the GPU's memory, a loop that cannot afford cudaMalloc's
device-wide synchronisation - so this entry point keeps its scratch in a fixed
array inside the library.  Its output must equal the ordinary entry point's,
on two calls in a row (the second call finds the scratch as the first left it).
This file sorts last on purpose: a run that stops at the first failure has then
run every other test."""
import ctypes
import math
from ctypes import c_double, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from rllm_b200.kernels import build
    lib = ctypes.CDLL(build.compile_library("attention_mma"))
    lib.rllm_attention_decode_workspace.restype = ctypes.c_longlong
    return lib


def _case(seed, lens, nq=8, nkv=2, d=64, page=16):
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    pages = sum(-(-n // page) for n in lens) + 4
    kc = torch.randn(pages, nkv, page, d, generator=g).bfloat16().to(DEV)
    vc = torch.randn(pages, nkv, page, d, generator=g).bfloat16().to(DEV)
    maxb = max(-(-n // page) for n in lens)
    table = torch.full((S, maxb), -1, dtype=torch.int32)
    perm = torch.randperm(pages, generator=g).tolist()
    for s, n in enumerate(lens):
        for b in range(-(-n // page)):
            table[s, b] = perm.pop()
    qkv = torch.randn(S, (nq + 2 * nkv) * d, generator=g).bfloat16().to(DEV)
    inv = torch.tensor([10000.0 ** (-(2 * i) / d) for i in range(d // 2)], dtype=torch.float64, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return dict(S=S, nq=nq, nkv=nkv, d=d, page=page, pages=pages, kc=kc, vc=vc, table=table.to(DEV), qkv=qkv,
                inv=inv, seq_lens=seq_lens, max_len=max(lens))


def _call(lib, fn_name, c, kc, vc, out, err, extra, window=0, write_kv=1):
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: c_void_p(t.data_ptr())
    fn = getattr(lib, fn_name)
    args = [p(c["qkv"]), c_int(c["qkv"].shape[1]), p(out), p(kc), p(vc), p(c["table"]), c_int(c["table"].shape[1]),
            p(c["seq_lens"]), c_int(c["S"]), c_int(c["max_len"]), c_int(c["nq"]), c_int(c["nkv"]), c_int(c["d"]),
            c_int(c["page"]), c_int(c["pages"]), c_int(window), c_float(1.0 / math.sqrt(c["d"])), p(c["inv"]),
            c_int(c["d"]), c_int(write_kv)] + extra + [p(err), stream]
    return fn(*args)


def test_allocation_free_decode_attention_matches_the_ordinary_one_twice():
    lib = _lib()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    for seed, lens in ((0, [1, 40, 129, 700, 1025]), (1, [300, 2, 511, 64, 128, 2049])):
        c = _case(seed, lens)
        # the ordinary entry point: the caller brings workspace and zeroed counters
        need = lib.rllm_attention_decode_workspace(c_int(c["S"]), c_int(c["nq"]), c_int(c["d"]), c_int(c["max_len"]))
        ws = torch.empty(need, dtype=torch.float32, device=DEV)
        counters = torch.zeros(c["S"] * c["nkv"], dtype=torch.int32, device=DEV)
        kc_a, vc_a = c["kc"].clone(), c["vc"].clone()
        out_a = torch.zeros(c["S"], c["nq"] * c["d"], dtype=torch.bfloat16, device=DEV)
        rc = _call(lib, "rllm_attention_decode_bf16", c, kc_a, vc_a, out_a, err,
                   [c_void_p(ws.data_ptr()), c_void_p(counters.data_ptr())])
        assert rc == 0
        # the allocation-free one: same inputs, nothing brought
        kc_b, vc_b = c["kc"].clone(), c["vc"].clone()
        out_b = torch.zeros_like(out_a)
        before = torch.cuda.memory_allocated()
        rc = _call(lib, "rllm_attention_decode_bf16_static", c, kc_b, vc_b, out_b, err, [])
        torch.cuda.synchronize()
        assert rc == 0 and torch.cuda.memory_allocated() == before
        assert int(err.item()) == 0
        assert float(out_a.abs().max()) > 0
        # same kernel, same arithmetic: within the bfloat16 tolerance of the kernel tests (in fact equal)
        diff = (out_a.float() - out_b.float()).abs().max() / out_a.float().abs().max()
        assert float(diff) <= 1.6e-2 and torch.equal(out_a, out_b)
        assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)      # the token's k and v were stored alike
        # and again at once: the scratch now holds what the call before left in it.  The device's free
        # memory, as the driver counts it, is the same after the call as before: nothing was allocated
        # behind PyTorch's back either (the first call above has loaded the module and its array).
        kc_c, vc_c = c["kc"].clone(), c["vc"].clone()
        out_c = torch.zeros_like(out_a)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(lib, "rllm_attention_decode_bf16_static", c, kc_c, vc_c, out_c, err, [])
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert rc == 0 and int(err.item()) == 0 and torch.equal(out_a, out_c)


def _plain_decode(c, window, write_kv):
    """The formula in float64 on the CPU: sequence s has one query at position len - 1 that sees keys
    max(0, len - window) .. len - 1 through its block table; q (and, with write_kv, the token's own key,
    which then comes from qkv and not from the cache) is rotated by the rotate-half rule."""
    nq, nkv, d, page = c["nq"], c["nkv"], c["d"], c["page"]
    qkv, kc, vc = c["qkv"].double().cpu(), c["kc"].double().cpu(), c["vc"].double().cpu()
    inv, table = c["inv"].cpu(), c["table"].cpu()
    out = torch.zeros(c["S"], nq * d, dtype=torch.float64)

    def rot(x, pos):
        a = pos * inv
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([x1 * torch.cos(a) - x2 * torch.sin(a), x2 * torch.cos(a) + x1 * torch.sin(a)], dim=-1)
    for s, n in enumerate(c["seq_lens"].tolist()):
        pos = n - 1
        q = rot(qkv[s, : nq * d].view(nq, d), pos)
        lo = max(0, n - window) if window else 0
        rows = [(int(table[s, j // page]), j % page) for j in range(lo, n)]
        k = torch.stack([kc[pg, :, r] for pg, r in rows])            # [keys, nkv, d]
        v = torch.stack([vc[pg, :, r] for pg, r in rows])
        if write_kv:
            k[-1] = rot(qkv[s, nq * d:(nq + nkv) * d].view(nkv, d), pos).bfloat16().double()
            v[-1] = qkv[s, (nq + nkv) * d:].view(nkv, d)
        for h in range(nq):
            kv = h // (nq // nkv)
            p = torch.softmax((k[:, kv] @ q[h]) / math.sqrt(d), dim=0)
            out[s, h * d:(h + 1) * d] = p @ v[:, kv]
    return out


@pytest.mark.parametrize("window,write_kv", [(100, 1), (0, 0), (37, 0)])
def test_allocation_free_decode_attention_with_a_window_and_without_the_cache_write(window, write_kv):
    """The same entry point with a sliding window, and reading the token's own key from the cache instead of
    storing it, against the formula in float64."""
    lib = _lib()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    c = _case(5 + window, [1, 36, 37, 38, 130, 600])
    kc, vc = c["kc"].clone(), c["vc"].clone()
    out = torch.zeros(c["S"], c["nq"] * c["d"], dtype=torch.bfloat16, device=DEV)
    rc = _call(lib, "rllm_attention_decode_bf16_static", c, kc, vc, out, err, [], window=window, write_kv=write_kv)
    torch.cuda.synchronize()
    assert rc == 0 and int(err.item()) == 0
    want = _plain_decode(c, window, write_kv)
    diff = (out.double().cpu() - want).abs().max() / want.abs().max()
    assert float(diff) <= 1.6e-2, float(diff)
    if not write_kv:
        assert torch.equal(kc, c["kc"]) and torch.equal(vc, c["vc"])      # nothing was stored


def test_sizes_beyond_the_fixed_scratch_are_refused():
    lib = _lib()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    c = _case(2, [64] * 4)
    out = torch.full((c["S"], c["nq"] * c["d"]), 7.0, dtype=torch.bfloat16, device=DEV)
    c["max_len"] = 64 * 1024 * 1024          # a bound on the lengths that needs far more scratch than the library holds
    rc = _call(lib, "rllm_attention_decode_bf16_static", c, c["kc"], c["vc"], out, err, [])
    torch.cuda.synchronize()
    assert rc == -3 and float(out.float().min()) == 7.0   # refused with its own code; nothing was launched
