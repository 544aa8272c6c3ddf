"""The custom-op registration of the vLLM-style hook, checked without a GPU: schema, the
mutated-buffer annotation and the shape-only (Meta) implementation used while tracing."""
import torch


def test_register_defines_op_with_meta_impl():
    from transarch_b200 import vllm_hook
    vllm_hook.register()
    vllm_hook.register()                                   # idempotent
    op = torch.ops.b200dsa.misa_sparse_attn_indexer
    schema = op.default._schema
    names = [a.name for a in schema.arguments]
    assert names[:7] == ["hidden_states", "k_cache_prefix", "kv_cache", "q_fp8", "k", "weights",
                         "q_head_topk_indices"]
    assert names[-1] == "topk_indices_buffer"
    assert schema.arguments[-1].alias_info is not None and schema.arguments[-1].alias_info.is_write
    assert all(a.alias_info is None for a in schema.arguments[:-1])       # nothing else is mutated
    T = 5
    m = lambda *s, dt=torch.bfloat16: torch.empty(*s, dtype=dt, device="meta")
    buf = m(T, 2048, dt=torch.int32)
    out = op(m(T, 7168), "model.layers.0.self_attn.indexer.k_cache", m(4, 64, 132, dt=torch.uint8),
             m(T, 64, 128, dt=torch.float8_e4m3fn), m(T, 128), m(T, 64, dt=torch.float32), None, 128, "ue8m0",
             8, 8, False, 1024, 8192, 2048, 128, 65536, 0, buf)
    assert out.shape == buf.shape and out.dtype == torch.int32 and out.device.type == "meta"


def test_hook_classes_mirror_reference_constructor():
    import inspect
    from transarch_b200 import vllm_hook
    params = list(inspect.signature(vllm_hook.MiSASparseAttnIndexer.__init__).parameters)[1:]
    assert params == ["k_cache", "quant_block_size", "scale_fmt", "topk_heads", "decode_topk_heads", "use_qnorm",
                      "k_block_size", "stage1_topk", "topk_tokens", "head_dim", "max_model_len",
                      "max_total_seq_len", "topk_indices_buffer"]
    # the reference's positional arguments first; anything after them (the metadata a caller may
    # pass when there is no vLLM forward context) must be optional
    sig = inspect.signature(vllm_hook.MiSASparseAttnIndexer.forward_cuda).parameters
    fwd = list(sig)[1:]
    assert fwd[:5] == ["hidden_states", "q_fp8", "k", "weights", "q_head_topk_indices"]
    assert all(sig[n].default is not inspect.Parameter.empty for n in fwd[5:])
    sig = inspect.signature(vllm_hook.BaselineSparseAttnIndexer.forward_cuda).parameters
    base = list(sig)[1:]
    assert base[:4] == ["hidden_states", "q_fp8", "k", "weights"]
    assert all(sig[n].default is not inspect.Parameter.empty for n in base[4:])
