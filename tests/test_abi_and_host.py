"""CPU-only checks of the drop-in boundary and the host logic: the shared library loads and
exports every symbol the public headers declare (no compute call is made), the ctypes
struct layouts match the reference's, and the paging helpers follow the pool's row rule."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "granite4_b200.h")
HEADER_CPP = os.path.join(ROOT, "include", "granite4_b200.hpp")


@pytest.fixture(scope="module")
def g4():
    import granite4_b200
    from granite4_b200 import _build
    if _build.is_stale():
        _build.build()
    return granite4_b200


def declared_c_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(granite4_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_c_functions()
    for must in ("granite4_kernel_rmsnorm", "granite4_prefill_embed_rows",
                 "granite4_prefill_rope_split_append_int8", "granite4_prefill_silu_mul",
                 "granite4_gpu_multi_rope_append", "granite4_kernel_add_rmsnorm_fp8",
                 "granite4_kernel_swiglu_fp8", "granite4_kernel_rope_kv_int8_paged",
                 "granite4_status", "granite4_get_model_info"):
        assert must in names


def test_library_exports_every_declared_symbol(g4):
    from granite4_b200 import capi
    dll = C.CDLL(g4._build.LIB_PATH)
    for name in declared_c_functions():
        assert hasattr(dll, name), f"{name} declared in the header but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == declared_c_functions()


def test_cpp_entry_points_keep_the_reference_mangled_names(g4):
    # what engine/src/forward_gpu.cu links against: namespace granite4, the reference's signatures
    out = subprocess.run(["nm", "-D", "--defined-only", g4._build.LIB_PATH], capture_output=True,
                         text=True, check=True).stdout
    for sym in ("_ZN8granite418prefill_embed_rowsEPKiiiPKtfPti",
                "_ZN8granite430prefill_rope_split_append_int8EPKtPKfS3_iiiiiiPtPaS5_PfS6_PKi",
                "_ZN8granite416prefill_silu_mulEPKfiiPt",
                "_ZN8granite421gpu_multi_rope_appendEPKtS1_S1_PKfS3_PKNS_12GpuMultiRowsEiiiiiPvS7_PfS8_iPt",
                "_ZN8granite414gpu_multi_ropeEPKtPKfS3_PKNS_12GpuMultiRowsEiiiPt",
                "_ZN8granite419gpu_multi_kv_appendEPKtS1_iPvS2_PfS3_PKNS_12GpuMultiRowsEiiii",
                "_ZN8granite425prefill_rope_split_appendEPKtPKfS3_iiiiiiPtS4_S4_PKi",
                "_ZN8granite417prefill_attentionEPKtS1_S1_fiiiiiiPtPKaS4_PKfS6_bPKhS8_bPKibi"):
        assert sym in out
    hpp = open(HEADER_CPP).read()
    for fn in ("prefill_embed_rows", "prefill_rope_split_append_int8", "prefill_silu_mul",
               "gpu_multi_rope_append", "gpu_multi_rope(", "gpu_multi_kv_append", "prefill_rope_split_append(",
               "prefill_attention("):
        assert fn in hpp


def test_model_info_and_status_without_compute(g4):
    from granite4_b200 import capi
    lib = capi.lib()
    info = lib.model_info()
    assert info.model_id == b"granite-4.2-8b" and info.gpu_target == b"sm_100a"
    assert (info.num_layers, info.hidden_size, info.intermediate_size) == (40, 4096, 12800)
    assert (info.num_attention_heads, info.num_key_value_heads, info.head_dim) == (32, 8, 128)
    assert (info.vocab_size, info.max_context_length) == (100352, 131072)
    st = lib.status()
    assert st.status == 1 and st.status_text == b"unimplemented"  # as the reference reports
    assert st.cuda_device_present in (0, 1)
    lib.granite4_get_model_info(None)  # NULL-tolerant like the reference
    lib.granite4_status(None)


def test_struct_layouts(g4):
    from granite4_b200 import capi
    # frontend/engine_bridge.py:45-51 binds {int, int, char*, char*}
    assert C.sizeof(capi.StatusInfo) == 24
    # engine/src/forward_gpu_api.h:162-182 on LP64
    expect = 4 + 16 * 4 + 4 + 16 * 8 + 16 * 8 + 16 * 4 + 4 + 16 * 4 + 16 * 4 + 16 * 8 * 4
    assert C.sizeof(capi.MultiRows) == expect + (8 - expect % 8) % 8
    assert capi.MultiRows.pt.offset == 72 and capi.MultiRows.tree.offset == 72 + 256 + 64


def test_invalid_arguments_are_refused_before_any_launch(g4, capfd):
    """The launchers validate first (engine/src/kernels_phase2.cu:912-915 style), so these
    calls return -1 without touching a device - they run on a machine with no GPU."""
    from granite4_b200 import capi
    lib = capi.lib()
    assert lib.granite4_kernel_rmsnorm(None, None, 1e-5, 1, 8, None) == -1
    assert lib.granite4_kernel_rmsnorm(16, 16, 0.0, 1, 8, 16) == -1          # eps must be > 0
    assert lib.granite4_kernel_rmsnorm(16, 16, 1e-5, 1 << 20, 1 << 12, 16) == -1  # rows*cols > INT_MAX
    assert lib.granite4_kernel_rmsnorm_batched(16, 16, 1e-5, 17, 8, 16) == -1   # rows <= 16
    assert lib.granite4_prefill_embed_rows(16, 0, 0, 16, 1.0, 16, 4096) == -1
    assert lib.granite4_prefill_embed_rows(16, 0, 65536, 16, 1.0, 16, 4096) == -1
    assert lib.granite4_prefill_silu_mul(16, 0, 4, 16) == -1
    assert lib.granite4_prefill_rope_split_append_int8(16, 16, 16, 0, 4, 32, 8, 64, 16, 16, 16, 16, 16,
                                                       16, None) == -1       # d must be 128
    assert lib.granite4_prefill_rope_split_append_int8(16, 16, 16, 10, 8, 32, 8, 128, 16, 16, 16, 16, 16,
                                                       16, None) == -1       # stride < base_pos + rows
    assert lib.granite4_gpu_multi_rope_append(16, 16, 16, 16, 16, None, 1, 32, 8, 128, 8, 16, 16, 16, 16,
                                              64, 16) == -1
    assert lib.granite4_gpu_multi_rope_append(16, 16, 16, 16, 16, 16, 17, 32, 8, 128, 8, 16, 16, 16, 16,
                                              64, 16) == -1
    assert lib.granite4_gpu_multi_rope_append(16, 16, 16, 16, 16, 16, 1, 32, 8, 128, 4, 16, 16, 16, 16,
                                              64, 16) == -1                  # only int8 is built
    assert lib.granite4_kernel_add_rmsnorm_fp8(16, 0, 16, 0, 16, 1e-5, 0.22, 4, 4097, 16, None, None,
                                               None, None) == -1             # cols % 8
    assert lib.granite4_kernel_add_rmsnorm_fp8(16, 0, 16, 0, 16, 1e-5, 0.22, 4, 4096, None, None, 16,
                                               None, None) == -1             # fp8 needs scale buffer
    assert lib.granite4_kernel_add_rmsnorm_fp8(24, 0, 16, 0, 16, 1e-5, 0.22, 4, 4096, 16, None, None,
                                               None, None) == -1             # misaligned
    assert lib.granite4_kernel_swiglu_fp8(16, 16, 0, 100, 4, 12800, 16, None, None) == -1  # ld < I
    assert lib.granite4_kernel_swiglu_fp8(16, 16, 0, 12800, 4, 12800, None, None, None) == -1
    assert lib.granite4_kernel_rope_kv_int8_paged(16, 16, 16, None, 16, 4, 32, 8, 128, 64, 64, 0, 16, 16,
                                                  16, 16, 16) == -1
    assert lib.granite4_kernel_rope(16, 16, 16, 4, 127, 16) == -1
    assert lib.granite4_kernel_kv_append_int8_batched(16, 16, 16, 16, 16, 16, 0, 17, 64, 8, 128,
                                                      None) == -1
    assert lib.granite4_rope_tables_build(1e7, 127, 16, None, None) == -1
    assert lib.granite4_kernel_embed_gather(16, 0, 16, 100, 1.0, 16, 4096) == -1
    assert lib.granite4_kernel_fp8_quant(16, 7, 16, 16) == -1
    assert "granite4:" in capfd.readouterr().err  # one diagnostic line per refusal


def test_kernels_refuse_cpu_tensors(g4):
    import torch
    from granite4_b200 import kernels
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        kernels._p(x, torch.bfloat16)


def test_row_table_follows_the_pool_rule(g4):
    from granite4_b200 import paging
    # engine/src/kv_pool.cc:285-298: out[p] = page_id * B + p % B
    bt = [5, 2, 9]
    t = paging.row_table(bt, 40)
    assert t.dtype == np.int32 and len(t) == 40
    assert list(t[:3]) == [80, 81, 82] and t[15] == 95 and t[16] == 32 and t[39] == 9 * 16 + 7
    with pytest.raises(ValueError):
        paging.row_table(bt, 49)
    paging.validate_rows(t, 160)
    with pytest.raises(ValueError):
        paging.validate_rows(t, 100)
    with pytest.raises(ValueError):
        paging.validate_rows(np.array([1, 1]), 16)
    tables = paging.permuted_block_tables(4, 512, 7680, seed=0)
    flat = np.concatenate(tables)
    assert len(set(flat.tolist())) == 2048 and flat.max() < 7680
    pos, rows = paging.batch_rows(tables, [100, 5000, 60000, 122880], 8192)
    assert pos.shape == rows.shape == (32768,) and pos.max() == 122880 + 8191
    paging.validate_rows(rows, 7680 * 16)


def test_glue_byte_counts(g4):
    from granite4_b200 import glue
    s = glue.GraniteShapes()
    b = glue.bytes_per_row(s)
    assert b == {"embed": 16388, "add_rmsnorm_fp8": 28672, "rope_kv_int8": 23108,
                 "swiglu_fp8": 64000, "final_norm": 16384}
    assert glue.bytes_per_token(s) == 5794464


def test_a_plain_c99_program_includes_the_header_and_links_the_library(g4, tmp_path):
    """The boundary is a C ABI: a strict C99 translation unit includes include/granite4_b200.h,
    links libgranite4_b200.so and runs (only entry points that need no GPU)."""
    import shutil
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    lib_dir = os.path.dirname(g4._build.LIB_PATH)
    exe = str(tmp_path / "abi_smoke")
    src = os.path.join(ROOT, "tests", "c_abi", "abi_smoke.c")
    build = subprocess.run([cc, "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                            src, "-o", exe, "-L", lib_dir, "-lgranite4_b200", "-Wl,-rpath," + lib_dir],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "granite-4.2-8b sm_100a layers=40" in run.stdout
    assert "pool ok=1 rows 12 13 8 11 | 2" in run.stdout  # pages are handed out from the top of the free stack


def test_bench_condenses_a_profiler_launch_list_into_traffic_per_op(tmp_path):
    """bench.py's converter: one line per launch and metric in, DRAM bytes per op launch out
    (mean over the launches of each kernel, summed over the op's kernels), and the loader turns
    the written file back into bytes per token row."""
    import bench
    head = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size",' \
           '"Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'

    def line(i, kernel, metric, unit, value):
        return f'"{i}","1","python","h","{kernel}","1","7","(128, 1, 1)","(8, 1, 1)","0","10.0","x","{metric}","{unit}","{value}"\n'
    stats = "void unnamed>::add_rmsnorm_fast_kernel<1, 1>(unnamed>::NormParams)"
    enc = "void unnamed>::norm_encode_kernel<1>(unnamed>::NormParams)"
    fin = "void unnamed>::add_rmsnorm_fast_kernel<0, 0>(unnamed>::NormParams)"
    text = "==PROF== Connected\n" + head
    text += line(0, stats, "dram__bytes_read.sum", "Mbyte", "100") + line(0, stats, "dram__bytes_write.sum", "byte", "50,000,000")
    text += line(1, enc, "dram__bytes_read.sum", "byte", "10000000") + line(1, enc, "dram__bytes_write.sum", "byte", "30000000")
    text += line(2, stats, "dram__bytes_read.sum", "byte", "120000000") + line(2, stats, "dram__bytes_write.sum", "byte", "50000000")
    text += line(2, stats, "gpu__time_duration.sum", "ns", "31040")
    text += line(3, fin, "dram__bytes_read.sum", "byte", "64") + line(3, fin, "dram__bytes_write.sum", "byte", "36")
    src, dst = tmp_path / "launches.csv", tmp_path / "traffic.txt"
    src.write_text(text)
    ops = bench.traffic_from_ncu(str(src), 1000, str(dst))
    assert ops == {"add_rmsnorm_fp8": 160e6 + 40e6, "final_norm": 100.0}
    old = bench.TRAFFIC_FILE
    bench.TRAFFIC_FILE = str(dst)
    try:
        assert bench.load_traffic() == {"add_rmsnorm_fp8": 200e3, "final_norm": 0.1}
    finally:
        bench.TRAFFIC_FILE = old
