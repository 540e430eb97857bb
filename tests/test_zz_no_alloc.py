"""The allocation-free dispatch entry point, called through its exported C symbol.

Callers that may not allocate device memory (they run inside someone else's memory pool, or while the allocator
is locked) use ``ep_dispatch_one_rank_noalloc``: its scratch is a fixed array inside the library.  The test loads
the shared object with ctypes, runs the entry point twice in a row on caller-provided buffers and checks that
every output is bit-identical to what ``ElasticBuffer.dispatch`` returns for a group of one rank."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, x, idx, w, E, quantize, outs, num_sms=8):
    T, H = x.shape
    K = idx.shape[1]
    err = ctypes.create_string_buffer(256)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.ep_dispatch_one_rank_noalloc(
        p(x), p(idx), p(w), T, H, K, E, int(quantize), p(outs['x']), p(outs['sf']), p(outs['idx']), p(outs['w']),
        p(outs['meta']), p(outs['lane_src']), p(outs['plan']), p(outs['psum_rank']), p(outs['psum_expert']),
        p(outs['per_expert']), num_sms, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    assert rc == 0, err.value.decode()


@pytest.mark.parametrize('quantize', [True, False])
def test_noalloc_dispatch_matches_elastic_buffer(quantize):
    from deepep_ascend_b200 import ElasticBuffer, _native
    _native.load()
    lib = ctypes.CDLL(_native.shared_object())
    lib.ep_dispatch_one_rank_noalloc.restype = ctypes.c_int
    T, H, E, K = 300, 1024, 16, 4
    G = H // 128
    dev = 'cuda'
    outs = {'x': torch.zeros(T, H, dtype=torch.float8_e4m3fn if quantize else torch.bfloat16, device=dev),
            'sf': torch.zeros(T, G, device=dev), 'idx': torch.zeros(T, K, dtype=torch.int64, device=dev),
            'w': torch.zeros(T, K, device=dev), 'meta': torch.zeros(T, 2, dtype=torch.int32, device=dev),
            'lane_src': torch.zeros(T, K, dtype=torch.int32, device=dev), 'plan': torch.zeros(T, K, dtype=torch.int32, device=dev),
            'psum_rank': torch.zeros(1, dtype=torch.int32, device=dev), 'psum_expert': torch.zeros(E, dtype=torch.int32, device=dev),
            'per_expert': torch.zeros(E, dtype=torch.int32, device=dev)}
    buf = ElasticBuffer(None, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=quantize)
    try:
        for call in range(2):            # two calls in a row share the built-in scratch array
            g = torch.Generator().manual_seed(100 + call)
            x = torch.randn(T, H, generator=g).bfloat16().cuda()
            idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices
            idx[torch.rand(idx.shape, generator=g) < 0.3] = -1
            idx[7] = -1                   # a token that goes nowhere
            idx = idx.cuda()
            w = torch.rand(T, K, generator=g).cuda()
            for t in outs.values():
                t.view(torch.uint8).fill_(0xEE)
            _call(lib, x, idx, w, E, quantize, outs)
            torch.cuda.synchronize()
            # the kernel's own verdict is readable without any allocation either
            status = (ctypes.c_ulonglong * 6)(*([7] * 6))
            err = ctypes.create_string_buffer(256)
            assert lib.ep_noalloc_last_status(status, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256) == 0
            assert list(status) == [0, 0, 0, 0, 0, 0], list(status)
            ref_x, ref_idx, ref_w, handle, _ = buf.dispatch(x, idx, w, num_experts=E, num_sms=8)
            torch.cuda.synchronize()
            n = handle.num_recv_tokens
            assert int(outs['psum_rank'][0]) == n == int((idx >= 0).any(dim=1).sum())
            rx, rsf = ref_x if quantize else (ref_x, None)
            assert torch.equal(outs['x'][:n].view(torch.uint8), rx.view(torch.uint8))
            if quantize:
                assert torch.equal(outs['sf'][:n], rsf)
            assert torch.equal(outs['idx'][:n], ref_idx) and torch.equal(outs['w'][:n], ref_w)
            assert torch.equal(outs['meta'][:n], handle.recv_src_metadata)
            assert torch.equal(outs['lane_src'], handle.dst_buffer_slot_idx) and torch.equal(outs['plan'], handle.plan)
            assert torch.equal(outs['psum_expert'], handle.psum_num_recv_tokens_per_expert)
            assert torch.equal(outs['per_expert'], handle.num_unaligned_recv_tokens_per_expert)
            # rows past the received count were never written
            assert bool((outs['x'][n:].view(torch.uint8) == 0xEE).all())
    finally:
        buf.destroy()


def test_noalloc_rejects_sizes_beyond_the_builtin_array():
    from deepep_ascend_b200 import _native
    _native.load()
    lib = ctypes.CDLL(_native.shared_object())
    err = ctypes.create_string_buffer(256)
    t = torch.zeros(64, device='cuda')
    p = ctypes.c_void_p(t.data_ptr())
    rc = lib.ep_dispatch_one_rank_noalloc(p, p, p, 4, 128, 2, 4096, 0, p, p, p, p, p, p, p, p, p, p, 8, None, err, 256)
    assert rc != 0 and b'num_experts' in err.value
    rc = lib.ep_dispatch_one_rank_noalloc(p, p, p, 4, 128, 2, 8, 0, p, p, p, p, p, p, p, p, p, p, 1000, None, err, 256)
    assert rc != 0 and b'num_sms' in err.value
    # misaligned pointers are refused on the host (nothing is launched): 4-byte aligned ids, 2-byte aligned weights
    p4, p2 = ctypes.c_void_p(t.data_ptr() + 4), ctypes.c_void_p(t.data_ptr() + 2)
    rc = lib.ep_dispatch_one_rank_noalloc(p, p4, p, 4, 128, 2, 8, 0, p, p, p, p, p, p, p, p, p, p, 8, None, err, 256)
    assert rc != 0 and b'8-byte aligned' in err.value
    rc = lib.ep_dispatch_one_rank_noalloc(p, p, p2, 4, 128, 2, 8, 0, p, p, p, p, p, p, p, p, p, p, 8, None, err, 256)
    assert rc != 0 and b'4-byte aligned' in err.value
