"""Routing-score generators (precise hot-rank ratio, Zipf skew) and the exact public surface of the package and of the
native module (a rename or a dropped binding fails here, on the CPU tier)."""
import torch


def test_precise_unbalanced_scores_hit_the_requested_ratio():
    from deepep_ascend_b200.utils import gate
    torch.manual_seed(0)
    checked = 0
    for per_rank in (1, 4, 8):
        for num_ranks in (2, 4, 8, 16):
            E = per_rank * num_ranks
            for K in (1, 2, 4, 6, 8):
                if K > E:
                    continue
                for ratio in (1.0, 2.0, 4.0):
                    lo = max(1, -(-K // per_rank))
                    hi = min(K, num_ranks, int((num_ranks - 1) / ratio) + 1)
                    if lo > hi:
                        continue
                    total = torch.zeros(num_ranks)
                    for _ in range(num_ranks):
                        s = gate.get_unbalanced_scores(4096, E, num_ranks, K, ratio, True, device='cpu')
                        idx = s.topk(K, dim=-1).indices
                        total += gate.rank_hit_counts(idx, E, num_ranks).float()
                    got = total[0].item() / max(total[1:].min().item(), 1)
                    spread = total[1:].max().item() / max(total[1:].min().item(), 1)
                    assert abs(got - ratio) / ratio < 0.1 and spread < 1.02, (per_rank, num_ranks, K, ratio, got, spread)
                    checked += 1
    assert checked > 50


def test_random_unbalanced_and_zipf_scores_are_skewed():
    from deepep_ascend_b200.utils import gate
    torch.manual_seed(1)
    s = gate.get_unbalanced_scores(4096, 64, 8, 4, 3.0, False, device='cpu')
    c = gate.rank_hit_counts(s.topk(4, dim=-1).indices, 64, 8).float()
    assert 2.0 < c[0] / c[1:].mean() < 4.5
    z = gate.get_zipf_scores(8192, 64, 1.2, device='cpu')
    first = (z.topk(6, dim=-1).indices == 0).any(dim=1).float().mean()
    last = (z.topk(6, dim=-1).indices == 63).any(dim=1).float().mean()
    assert first > 0.6 and last < 0.1
    b = gate.get_balanced_scores(4096, 64, device='cpu')
    cb = gate.rank_hit_counts(b.topk(4, dim=-1).indices, 64, 8).float()
    assert cb.max() / cb.min() < 1.15


PACKAGE_EXPORTS = ['Buffer', 'Config', 'EPHandle', 'ElasticBuffer', 'EventHandle', 'EventOverlap', 'get_logical_domain_size',
                   'get_physical_domain_size', 'topk_idx_t']
BUFFER_METHODS = ['all_gather', 'barrier', 'capture', 'combine', 'destroy', 'dispatch', 'engram_fetch', 'engram_write',
                  'get_buffer_size_hint', 'get_comm_stream', 'get_theoretical_num_sms', 'low_latency_combine', 'low_latency_dispatch',
                  'pp_recv', 'pp_send', 'pp_set_config', 'get_dispatch_layout', 'get_combine_buffer', 'reduce_scatter',
                  'create_agrs_session', 'destroy_agrs_session', 'agrs_set_config', 'agrs_get_inplace_tensor',
                  'low_latency_update_mask_buffer', 'low_latency_query_mask_buffer', 'low_latency_clean_mask_buffer',
                  'get_next_low_latency_combine_buffer', 'get_physical_domain_size', 'get_logical_domain_size']
NATIVE_FUNCTIONS = ['ag_gemm', 'dequant_transpose', 'expert_segments', 'gemm_error', 'gemm_kgrouped', 'gemm_nt', 'gemm_rs', 'get_dispatch_layout',
                    'get_elastic_buffer_alignment', 'get_platform', 'get_workspace_bytes', 'local_expand_copy', 'local_expand_plan',
                    'local_reduce', 'moe_bwd_prep', 'per_token_cast_to_fp8',
                    'swiglu_bwd', 'swiglu_quant', 'weighted_transpose']
NATIVE_CLASSES = ['CombineCall', 'DispatchCall', 'ElasticBuffer', 'RecvSlot', 'LLCombineCall', 'LLDispatchCall', 'MoeShape', 'RegionLayout']


def test_public_surface():
    import deepep_ascend_b200 as ep
    for name in PACKAGE_EXPORTS:
        assert hasattr(ep, name), name
    for name in BUFFER_METHODS:
        assert callable(getattr(ep.ElasticBuffer, name, None)), name
    for name in ('dispatch', 'combine', 'get_dispatch_layout', 'low_latency_dispatch', 'low_latency_combine',
                 'clean_low_latency_buffer', 'get_next_low_latency_combine_buffer', 'sync', 'get_local_ipc_handle',
                 'get_local_buffer_tensor', 'get_local_device_id', 'get_comm_stream', 'is_available'):
        assert callable(getattr(ep.Buffer, name, None)), name
    handle_fields = ['do_expand', 'num_experts', 'expert_alignment', 'num_max_tokens_per_rank', 'num_sms', 'topk_idx', 'num_recv_tokens',
                     'num_expanded_tokens', 'psum_num_recv_tokens_per_scaleup_rank', 'psum_num_recv_tokens_per_expert',
                     'num_unaligned_recv_tokens_per_expert', 'recv_src_metadata', 'dst_buffer_slot_idx']
    import inspect
    params = inspect.signature(ep.EPHandle.__init__).parameters
    for f in handle_fields:
        assert f in params, f


def test_native_module_surface():
    from deepep_ascend_b200 import _native
    C = _native.load()
    assert C.get_platform() == 'cuda-sm100a'
    for name in NATIVE_FUNCTIONS:
        assert callable(getattr(C, name, None)), name
    for name in NATIVE_CLASSES:
        assert isinstance(getattr(C, name, None), type), name
    assert C.MAX_RANKS == 8 and C.MAX_TOPK == 16 and C.MAX_EXPERTS == 1024
    assert C.get_workspace_bytes() == 4 << 20


def test_native_surface_names_of_the_reference():
    """Every name of the reference's native-module contract (tests/platform/api_contract.py:1-42) resolves on the ``_C``
    facade, on the buffer classes and on the event handle; the JIT and NCCL-communicator hooks are inert."""
    from deepep_ascend_b200 import _C
    for name in ('get_platform', 'topk_idx_t', 'EventHandle', 'ElasticBuffer', 'calculate_elastic_buffer_size', 'is_sm90_compiled',
                 'init_jit', 'Config', 'Buffer', 'get_low_latency_rdma_size_hint', 'create_cpu_handle', 'get_elastic_buffer_alignment',
                 'get_local_nccl_unique_id', 'create_nccl_comm', 'destroy_nccl_comm', 'get_physical_domain_size',
                 'get_logical_domain_size'):
        assert getattr(_C, name, None) is not None, name
    assert _C.is_sm90_compiled() is False and _C.init_jit('/nowhere', '/usr/local/cuda') is None
    assert _C.destroy_nccl_comm(_C.create_nccl_comm(_C.get_local_nccl_unique_id(), 0, 1)) is None
    assert isinstance(_C.create_cpu_handle(1 << 20), bytes)
    for name in ('destroy', 'get_comm_stream', 'get_physical_domain_size', 'get_logical_domain_size', 'barrier', 'dispatch', 'combine',
                 'engram_write', 'engram_fetch', 'pp_set_config', 'pp_send', 'pp_recv', 'create_agrs_session', 'destroy_agrs_session',
                 'agrs_set_config', 'agrs_get_inplace_tensor', 'all_gather'):
        import deepep_ascend_b200 as ep
        assert callable(getattr(ep.ElasticBuffer, name, None)), name
    for name in ('is_available', 'get_num_rdma_ranks', 'get_rdma_rank', 'get_root_rdma_rank', 'get_local_device_id', 'get_local_ipc_handle',
                 'get_local_nvshmem_unique_id', 'get_local_buffer_tensor', 'get_comm_stream', 'sync', 'destroy', 'get_dispatch_layout',
                 'intranode_dispatch', 'intranode_combine', 'internode_dispatch', 'internode_combine', 'clean_low_latency_buffer',
                 'low_latency_dispatch', 'low_latency_combine', 'low_latency_update_mask_buffer', 'low_latency_query_mask_buffer',
                 'low_latency_clean_mask_buffer', 'get_next_low_latency_combine_buffer'):
        assert callable(getattr(_C.Buffer, name, None)), name
    assert callable(_C.Config.get_nvl_buffer_size_hint) and callable(_C.Config.get_rdma_buffer_size_hint)
    assert callable(_C.EventHandle.current_stream_wait)


def test_persistent_envs_are_captured_and_applied(tmp_path, monkeypatch):
    """Variables fixed at build time come back at import unless the process sets them itself."""
    import json
    import os
    from deepep_ascend_b200 import _native
    (tmp_path / 'persistent_envs.json').write_text(json.dumps({'EP_NUM_TOPK_IDX_BITS': '32', 'SOMETHING_ELSE': '1'}))
    monkeypatch.delenv('EP_NUM_TOPK_IDX_BITS', raising=False)
    monkeypatch.delenv('SOMETHING_ELSE', raising=False)
    assert _native.apply_persistent_envs(str(tmp_path))['EP_NUM_TOPK_IDX_BITS'] == '32'
    assert os.environ['EP_NUM_TOPK_IDX_BITS'] == '32' and 'SOMETHING_ELSE' not in os.environ      # only the listed names
    monkeypatch.setenv('EP_NUM_TOPK_IDX_BITS', '64')
    _native.apply_persistent_envs(str(tmp_path))
    assert os.environ['EP_NUM_TOPK_IDX_BITS'] == '64'                                              # the process wins
    assert _native.apply_persistent_envs(str(tmp_path / 'missing')) == {}
