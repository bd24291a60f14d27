"""CPU-only checks of the C-ABI boundary: the library builds/loads and exports every symbol
include/ctdk.h declares; argument validation errors come back as status codes with messages."""
import ctypes as C

from emberlm_b200 import lib


def test_library_exports_every_declared_symbol():
    names = lib.declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib.raw(), n)]
    assert missing == []


def test_ctypes_signature_table_covers_header():
    special = {"ctdk_last_error", "ctdk_sm_count", "ctdk_rmsnorm_bwd_scratch_floats",
               "ctdk_qk_norm_rope_bwd_scratch_floats", "ctdk_launch_count", "ctdk_prof_enable",
               "ctdk_prof_collect", "ctdk_gemm_3xtf32_workspace_floats", "ctdk_sample_workspace_bytes"}
    # engine / trainer / decoder entry points are bound in emberlm_b200/engine.py
    engine = {n for n in lib.declared_symbols()
              if n.startswith(("ctdk_engine_", "ctdk_model_", "ctdk_decode_", "ctdk_trainer_", "ctdk_dp_", "ctdk_batch_"))}
    from emberlm_b200 import engine as E
    assert all(getattr(E._L, n).argtypes is not None for n in engine if n.startswith(("ctdk_trainer_", "ctdk_dp_", "ctdk_batch_")))
    assert set(lib.declared_symbols()) - special - engine - set(lib._SIGS) == set()


def test_bad_arguments_return_einval_with_message():
    L = lib.raw()
    assert L.ctdk_add(None, None, None, -1, None) == lib.CTDK_EINVAL
    assert b"negative" in L.ctdk_last_error()
    assert L.ctdk_gemm(None, None, None, 4, 4, 4, 4, 4, 2, 0, 0, 0, 0, None, None) == lib.CTDK_EINVAL
    assert L.ctdk_attn_fwd(None, None, None, 1, 8, 3, 2, 64, None) == lib.CTDK_EINVAL
    assert L.ctdk_attn_fwd(None, None, None, 1, 8, 4, 2, 48, None) == lib.CTDK_EINVAL


def test_scratch_size_queries():
    L = lib.raw()
    assert L.ctdk_rmsnorm_bwd_scratch_floats(960) == 2048 * 960
    assert L.ctdk_qk_norm_rope_bwd_scratch_floats(128) == 512 * 2 * 128


def test_model_layout_matches_reference_parameter_counts():
    from emberlm_b200 import engine as E
    # parameter counts of the five presets (tied embeddings)
    want = {"smollm2_135m": (272, 134515008), "smollm2_360m": (290, 361821120),
            "qwen3_0_6b": (310, 596049920), "llama3_2_1b": (146, 1235814400),
            "qwen3_1_7b": (310, 1720574976)}
    for name, (ntens, nparam) in want.items():
        cfg = E.make_config(**E.PRESETS[name])
        lo = E.model_layout(cfg)
        assert len(lo.names) == ntens and sum(lo.numels) == nparam, name
        assert all(o % 64 == 0 for o in lo.offsets)
        # q,k,v and gate,up are adjacent (they run as one GEMM)
        i = lo.names.index("model.layers.0.self_attn.q_proj.weight")
        assert lo.offsets[i + 1] == lo.offsets[i] + lo.numels[i]
        assert lo.offsets[i + 2] == lo.offsets[i + 1] + lo.numels[i + 1]
        j = lo.names.index("model.layers.0.mlp.gate_proj.weight")
        assert lo.offsets[j + 1] == lo.offsets[j] + lo.numels[j]


def test_engine_rejects_bad_config():
    from emberlm_b200 import engine as E
    cfg = E.make_config(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                        num_attention_heads=3, num_key_value_heads=2, head_dim=64)
    assert E._L.ctdk_model_num_tensors(C.byref(cfg)) == -1
    assert "multiple of kv heads" in lib.last_error()
