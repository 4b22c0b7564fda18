"""GGUF container glue through the C ABI: the reference parser's own unit-test vectors
(src/parser.rs:209-303), a file with metadata and tensors, and (GPU) get_rows from a tensor
uploaded out of a GGUF file."""
import os
import struct

import numpy as np
import pytest

from agention_infer_b200 import AGN_Q4_K, AGN_Q8_0, _abi, synth
from agention_infer_b200.backend import BackendError
from agention_infer_b200.gguf import GgufError, GgufFile
from oracle import oracle as orc
from tests import gguf_writer as gw


def test_parse_minimal_v2():  # src/parser.rs:209-218
    g = GgufFile(data=gw.header(2, 0, 0))
    assert g.version == 2 and g.tensor_count == 0 and g.metadata_count == 0 and g.tensors() == []


def test_parse_invalid_magic():  # src/parser.rs:220-225
    with pytest.raises(GgufError) as e:
        GgufFile(data=bytes(24))
    assert e.value.status == _abi.AGN_EFORMAT and "magic" in str(e.value)


def test_parse_unsupported_version():  # src/parser.rs:227-233
    with pytest.raises(GgufError) as e:
        GgufFile(data=gw.header(1, 0, 0))
    assert "version 1" in str(e.value)
    with pytest.raises(GgufError):
        GgufFile(data=gw.header(4, 0, 0))


def test_parse_v3_with_metadata():  # src/parser.rs:235-246
    data = gw.header(3, 0, 1) + gw.gstr("general.architecture") + struct.pack("<I", 8) + gw.gstr("llama")
    g = GgufFile(data=data)
    assert g.version == 3 and g.get_string("general.architecture") == "llama"
    assert g.get_u64("general.architecture") is None and g.get_string("missing") is None


def test_parse_metadata_u32():  # src/parser.rs:248-257
    data = gw.header(3, 0, 1) + gw.gstr("test.value") + struct.pack("<II", 4, 42)
    assert GgufFile(data=data).get_u64("test.value") == 42


def test_parse_with_tensor():  # src/parser.rs:259-275
    data = gw.header(3, 1, 0) + gw.gstr("output.weight") + struct.pack("<IQQIQ", 2, 4096, 4096, 8, 0)
    g = GgufFile(data=data)
    (t,) = g.tensors()
    assert t.name == "output.weight" and t.dims == [4096, 4096] and t.ggml_type == AGN_Q8_0
    assert t.row_len == 4096 and t.n_rows == 4096 and t.row_bytes == 4352  # 128 blocks of 34 bytes
    assert g.data_offset % 32 == 0 and g.data_offset >= len(data)


def test_parse_array_metadata():  # src/parser.rs:277-294
    data = gw.header(3, 0, 1) + gw.gstr("tokenizer.ggml.bos_token_id") + struct.pack("<IIQI", 9, 4, 1, 1)
    assert GgufFile(data=data).get_array_info("tokenizer.ggml.bos_token_id") == (4, 1)


def test_unexpected_eof():  # src/parser.rs:296-303
    with pytest.raises(GgufError) as e:
        GgufFile(data=gw.header(3, 0, 1))
    assert e.value.status == _abi.AGN_EFORMAT and "end of data" in str(e.value)


def test_unknown_types_are_errors():
    with pytest.raises(GgufError) as e:  # `UnknownMetadataType`
        GgufFile(data=gw.header(3, 0, 1) + gw.gstr("k") + struct.pack("<II", 13, 0))
    assert "metadata type 13" in str(e.value)
    with pytest.raises(GgufError):  # `GgmlType::from_u32` rejects the removed ids 4 and 5
        GgufFile(data=gw.header(3, 1, 0) + gw.gstr("t") + struct.pack("<IQIQ", 1, 32, 4, 0))


def _model_file(vocab=96, hidden=256):
    table = synth.quant_table(AGN_Q4_K, vocab, hidden, cfg_index=2)
    norm = synth.norm_weight(2, "w", hidden)
    meta = [("general.architecture", "str", "llama"), ("llama.embedding_length", "u32", hidden),
            ("llama.attention.layer_norm_rms_epsilon", "f32", 1e-5), ("llama.rope.freq_base", "f64", 500000.0),
            ("llama.block_count", "u64", 2), ("llama.context_length", "u16", 4096), ("general.flag", "bool", 1),
            ("tokenizer.ggml.tokens", "array", ("str", ["<s>", "</s>", "hello", "wor", "ld"])),
            ("tokenizer.ggml.scores", "array", ("f32", [0.0, -1.0, -2.5])), ("general.quant_version", "i32", -2)]
    tensors = [("token_embd.weight", AGN_Q4_K, [hidden, vocab], table), ("output_norm.weight", 0, [hidden], norm),
               ("blk.0.ffn_gate.weight", 11, [256, 4], bytes(110 * 4))]  # Q3_K: listed, but no codec here
    return gw.build(3, meta, tensors), table, norm


def _one_tensor_header(dims, ggml_type, byte_offset):
    return (gw.header(3, 1, 0) + gw.gstr("t") + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) +
            struct.pack("<IQ", ggml_type, byte_offset))


def test_crafted_sizes_and_offsets_are_format_errors_not_wrapped_numbers():
    """Sizes and offsets come from the file; the reference rejects them with checked slices
    (src/quant/mod.rs:124-131).  A product or sum that wraps around 64 bits must not come out as a
    small, plausible number."""
    # dims whose product wraps: 2^33 * 2^33 rows
    g = GgufFile(data=_one_tensor_header([256, 1 << 33, 1 << 33], AGN_Q8_0, 0))
    with pytest.raises(GgufError) as e:
        g.tensors()
    assert e.value.status == _abi.AGN_EFORMAT
    with pytest.raises(GgufError):
        g.find("t")
    # row_bytes * n_rows wraps although the row count itself fits
    g = GgufFile(data=_one_tensor_header([1 << 40, 1 << 30], AGN_Q8_0, 0))
    with pytest.raises(GgufError):
        g.find("t")
    # a row length that would wrap inside type_size
    g = GgufFile(data=_one_tensor_header([(1 << 64) - 1], AGN_Q4_K, 0))
    with pytest.raises(GgufError):
        g.find("t")
    # data_offset + byte_offset wraps
    g = GgufFile(data=_one_tensor_header([32, 2], AGN_Q8_0, (1 << 64) - 8))
    with pytest.raises(GgufError):
        g.find("t")
    # a byte_offset just below the wrap: the directory entry is readable, the bytes are not in the file
    g = GgufFile(data=_one_tensor_header([32, 2], AGN_Q8_0, (1 << 64) - 4096))
    t = g.find("t")
    assert t.n_bytes == 68 and t.file_offset > (1 << 63)


@pytest.mark.gpu
def test_upload_of_a_tensor_outside_the_file_is_rejected(backend):
    for off in ((1 << 64) - 4096, 1 << 40):
        g = GgufFile(data=_one_tensor_header([32, 2], AGN_Q8_0, off) + bytes(256))
        with pytest.raises(BackendError) as e:
            g.upload(backend, "t")
        assert e.value.status == _abi.AGN_EFORMAT


@pytest.mark.gpu
def test_get_rows_rejects_a_row_count_whose_byte_size_wraps(backend):
    t = backend.empty(4096); ids = backend.upload(np.zeros(1, np.uint32)); o = backend.empty(4 * 256)
    with pytest.raises(BackendError) as e:  # n_rows * 144 wraps to a small number
        backend.get_rows(AGN_Q4_K, t, 4096, (1 << 63) // 144 * 2 + 1, 256, ids, 1, out=o)
    assert e.value.status == _abi.AGN_EINVAL


def test_file_with_metadata_and_tensors(tmp_path):
    blob, table, norm = _model_file()
    path = tmp_path / "tiny.gguf"
    path.write_bytes(blob)
    for g in (GgufFile(str(path)), GgufFile(data=blob)):
        assert g.metadata_count == 10 and g.tensor_count == 3
        assert g.get_u64("llama.embedding_length") == 256 and g.get_u64("llama.block_count") == 2
        assert g.get_u64("llama.context_length") == 4096 and g.get_u64("general.quant_version") is None  # signed: not a u64
        assert abs(g.get_f32("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
        assert g.get_f32("llama.rope.freq_base") == 500000.0  # Float64 narrows
        assert g.get_array_info("tokenizer.ggml.tokens") == (8, 5) and g.get_array_info("tokenizer.ggml.scores") == (6, 3)
        assert g.get_i64_array("tokenizer.ggml.scores") is None and g.get_i64_array("tokenizer.ggml.tokens") is None  # not integers
        emb = g.find("token_embd.weight")
        assert emb.dims == [256, 96] and emb.row_len == 256 and emb.n_rows == 96 and emb.row_bytes == 144
        assert emb.file_offset == g.data_offset + emb.byte_offset and emb.file_offset % 32 == 0
        assert blob[emb.file_offset:emb.file_offset + emb.n_bytes] == table.tobytes()
        nw = g.find("output_norm.weight")
        assert nw.n_rows == 1 and nw.row_len == 256 and nw.n_bytes == 1024
        assert np.array_equal(np.frombuffer(blob[nw.file_offset:nw.file_offset + 1024], np.float32), norm)
        assert g.find("blk.0.ffn_gate.weight").row_bytes == 0 and g.find("nope") is None
        g.close()
    with pytest.raises(GgufError) as e:
        GgufFile(str(tmp_path / "absent.gguf"))
    assert e.value.status == _abi.AGN_EIO


def test_rope_freq_scale_reference_vectors():  # src/model/llama/cpu_path.rs:1034-1060, the product's own host function
    from agention_infer_b200.gguf import rope_freq_scale as scale
    assert scale(None, None) == 1.0 and scale("none", 8.0) == 1.0 and scale("", 8.0) == 1.0
    assert scale("linear", 4.0) == 0.25 and scale("linear", 2.0) == 0.5 and scale("linear", None) == 1.0
    assert scale("yarn", 4.0) is None
    assert scale("linear", 0.0) == pytest.approx(1e6, rel=1e-6)  # factor.max(1e-6): no division by zero


def test_model_config_from_metadata():  # src/model/mod.rs:213-286
    table = synth.quant_table(AGN_Q4_K, 96, 256, cfg_index=2)
    meta = [("general.architecture", "str", "llama"), ("llama.embedding_length", "u32", 256), ("llama.attention.head_count", "u32", 4),
            ("llama.attention.layer_norm_rms_epsilon", "f32", 1e-5), ("llama.rope.freq_base", "f64", 500000.0),
            ("llama.block_count", "u64", 2), ("llama.context_length", "u16", 4096)]
    blob = gw.build(3, meta, [("token_embd.weight", AGN_Q4_K, [256, 96], table)])
    cfg = GgufFile(data=blob).model_config()
    assert cfg.architecture == "llama" and cfg.embedding_length == 256 and cfg.block_count == 2 and cfg.context_length == 4096
    assert cfg.vocab_size == 96 and cfg.rope_freq_base == 500000.0 and abs(cfg.layer_norm_rms_epsilon - 1e-5) < 1e-12
    assert cfg.feed_forward_length == 0 and cfg.rope_scaling_type is None and cfg.freq_scale == 1.0
    # head_count is mandatory
    assert cfg.head_count == 4 and cfg.head_count_kv == 4 and cfg.head_dim == 64  # kv falls back to head_count, dim to H / heads
    meta = [("general.architecture", "str", "qwen3"), ("qwen3.embedding_length", "u32", 1024), ("qwen3.attention.head_count", "u32", 16),
            ("qwen3.attention.head_count_kv", "u32", 8), ("qwen3.attention.key_length", "u32", 128),
            ("qwen3.rope.scaling.type", "str", "linear"), ("qwen3.rope.scaling.factor", "f32", 4.0),
            ("qwen3.feed_forward_length", "u32", 3072)]
    with pytest.raises(GgufError):  # "missing metadata: llama.attention.head_count"
        GgufFile(data=_model_file()[0]).model_config()
    table = synth.quant_table(AGN_Q4_K, 32, 1024, cfg_index=2)
    cfg2 = GgufFile(data=gw.build(3, meta, [("token_embd.weight", AGN_Q4_K, [1024, 32], table)])).model_config()
    assert (cfg2.head_count, cfg2.head_count_kv, cfg2.head_dim, cfg2.feed_forward_length) == (16, 8, 128, 3072)
    assert cfg2.rope_freq_base == 10000.0 and cfg2.context_length == 4096 and cfg2.block_count == 32 and cfg2.freq_scale == 0.25
    # a per-layer head_count_kv array (LFM2: 0 for the short-conv layers): the largest positive entry
    meta3 = [("general.architecture", "str", "lfm2"), ("lfm2.embedding_length", "u32", 1024), ("lfm2.attention.head_count", "u32", 16),
             ("lfm2.attention.head_count_kv", "array", ("i32", [0, 0, 8, 0, 4, 8]))]
    g3 = GgufFile(data=gw.build(3, meta3, [("token_embd.weight", AGN_Q4_K, [1024, 32], table)]))
    assert g3.get_i64_array("lfm2.attention.head_count_kv") == [0, 0, 8, 0, 4, 8] and g3.get_i64_array("nope") is None
    assert g3.model_config().head_count_kv == 8
    with pytest.raises(GgufError):  # "missing metadata: general.architecture"
        GgufFile(data=gw.build(3, [("x.y", "u32", 1)], [("token_embd.weight", AGN_Q4_K, [1024, 32], table)])).model_config()


def test_split_index_reference_vectors():  # src/loader.rs:108-119
    from agention_infer_b200.gguf import split_index
    assert split_index("MiniMax-M2.7-UD-IQ4_XS-00001-of-00004.gguf") == (1, 4)
    assert split_index("model-00003-of-00005.gguf") == (3, 5)
    assert split_index("single.gguf") is None
    assert split_index("model-0000x-of-00005.gguf") is None and split_index("model-00001-of-00002.bin") is None


def test_split_model_maps_the_sibling_files(tmp_path):
    """File 1 holds the header and the first tensors, file 2 only tensor bytes; offsets run on
    (`MultiFileMmap::load` / `slice`, src/loader.rs:49-90)."""
    blob, table, norm = _model_file()
    g0 = GgufFile(data=blob)
    nw = g0.find("output_norm.weight")
    cut = nw.file_offset  # the norm weight and everything after it go to the second file
    (tmp_path / "m-00001-of-00002.gguf").write_bytes(blob[:cut])
    with pytest.raises(GgufError) as e:  # the sibling is missing
        GgufFile(str(tmp_path / "m-00001-of-00002.gguf"))
    assert e.value.status == _abi.AGN_EIO
    (tmp_path / "m-00002-of-00002.gguf").write_bytes(blob[cut:])
    g = GgufFile(str(tmp_path / "m-00001-of-00002.gguf"))
    assert g.tensor_count == 3 and g.find("output_norm.weight").file_offset == cut
    g.close(); g0.close()


@pytest.mark.gpu
def test_dequant_whole_tensor(backend):  # WeightMap::dequant_tensor, src/model/mod.rs:318-345
    blob, table, norm = _model_file(vocab=40, hidden=768)
    g = GgufFile(data=blob)
    out, info = g.dequant_tensor(backend, "token_embd.weight")
    st, ref = orc.get_rows(orc.Q4_K, table, 40, 768, np.arange(40, dtype=np.uint32))
    assert st == orc.OK and np.array_equal(backend.read(out, np.float32, (40, 768)).view(np.uint32), ref.view(np.uint32))
    out, info = g.dequant_tensor(backend, "output_norm.weight")
    assert np.array_equal(backend.read(out, np.float32, (768,)), norm)


@pytest.mark.gpu
def test_upload_from_a_split_model(backend, tmp_path):
    blob, table, norm = _model_file(vocab=64, hidden=512)
    g0 = GgufFile(data=blob)
    cut = g0.find("output_norm.weight").file_offset
    (tmp_path / "m-00001-of-00002.gguf").write_bytes(blob[:cut])
    (tmp_path / "m-00002-of-00002.gguf").write_bytes(blob[cut:])
    g = GgufFile(str(tmp_path / "m-00001-of-00002.gguf"))
    dtab, info = g.upload(backend, "token_embd.weight")       # lies in file 1
    assert backend.read(dtab, np.uint8, (info.n_bytes,)).tobytes() == table.tobytes()
    dnorm, ninfo = g.upload(backend, "output_norm.weight")    # lies in file 2
    assert np.array_equal(backend.read(dnorm, np.float32, (ninfo.row_len,)), norm)
    # a tensor cut in two by the file boundary cannot be served from one mapping
    cut2 = g0.find("token_embd.weight").file_offset + 1000
    (tmp_path / "n-00001-of-00002.gguf").write_bytes(blob[:cut2])
    (tmp_path / "n-00002-of-00002.gguf").write_bytes(blob[cut2:])
    g2 = GgufFile(str(tmp_path / "n-00001-of-00002.gguf"))
    from agention_infer_b200 import BackendError
    with pytest.raises(BackendError) as e:
        g2.upload(backend, "token_embd.weight")
    assert e.value.status == _abi.AGN_EFORMAT
    g.close(); g2.close(); g0.close()


@pytest.mark.gpu
def test_get_rows_from_a_tensor_uploaded_out_of_a_gguf_file(backend, tmp_path):
    blob, table, norm = _model_file(vocab=512, hidden=1024)
    path = tmp_path / "tiny.gguf"
    path.write_bytes(blob)
    g = GgufFile(str(path))
    dtab, info = g.upload(backend, "token_embd.weight")
    ids = synth.token_ids(2, 100, info.n_rows)
    out = backend.get_rows(info.ggml_type, dtab, info.n_bytes, info.n_rows, info.row_len, backend.upload(ids), 100)
    st, ref = orc.get_rows(orc.Q4_K, table, info.n_rows, info.row_len, ids)
    assert st == orc.OK and np.array_equal(backend.read(out, np.float32, ref.shape).view(np.uint32), ref.view(np.uint32))
    dnorm, ninfo = g.upload(backend, "output_norm.weight")
    assert np.array_equal(backend.read(dnorm, np.float32, (ninfo.row_len,)), norm)
    from agention_infer_b200 import BackendError
    with pytest.raises(BackendError) as e:
        g.upload(backend, "blk.0.ffn_gate.weight")
    assert e.value.status == _abi.AGN_EUNSUPPORTED_DTYPE
    with pytest.raises(BackendError) as e:
        g.upload(backend, "nope")
    assert e.value.status == _abi.AGN_ENOTFOUND


def _many_tensor_file(n_tensors=6, rows=64, hidden=4096):
    """A file with several Q8_0 tensors of 136 KiB each (33 pages), so that page release has whole pages to drop."""
    rng = np.random.default_rng(77)
    tensors, raw = [], {}
    for i in range(n_tensors):
        t = synth.quant_table(orc.Q8_0, rows, hidden, cfg_index=0)
        t = (t.astype(np.int32) + i).astype(np.uint8)  # distinct bytes per tensor
        raw[f"blk.{i}.attn_q.weight"] = t
        tensors.append((f"blk.{i}.attn_q.weight", orc.Q8_0, [hidden, rows], t))
    blob = gw.build(3, [("general.architecture", "str", "llama")], tensors)
    return bytes(blob), raw


def test_release_pages_drops_whole_pages_and_data_stays_readable(tmp_path):  # release_mmap_prefix, gpu_resident.rs:29-49
    blob, raw = _many_tensor_file()
    path = tmp_path / "many.gguf"
    path.write_bytes(blob)
    g = GgufFile(str(path))
    page = os.sysconf("SC_PAGESIZE")
    infos = [g.find(n) for n in raw]
    lo, hi = infos[1].file_offset + 5, infos[3].file_offset + infos[3].n_bytes - 7  # deliberately unaligned
    want = hi // page * page - -(-lo // page) * page
    assert want > 0
    assert g.release_pages(lo, hi) == want
    assert g.release_pages(hi, lo) == 0 and g.release_pages(lo, lo + 10) == 0  # empty range, no whole page inside
    assert g.release_pages(0, 1 << 62) == len(blob) // page * page  # clipped to the file
    for n, info in zip(raw, infos):  # every tensor still reads back from the mapping (pages re-fault from the file)
        assert g.tensor_bytes(n) == raw[n].tobytes()
    g2 = GgufFile(data=blob)  # memory of the caller: nothing to release
    assert g2.release_pages(lo, hi) == 0
    g.close(); g2.close()


@pytest.mark.gpu
def test_upload_tensors_in_file_order_with_page_release(backend, tmp_path):  # pre_upload_gpu, gpu_resident.rs:112-152
    blob, raw = _many_tensor_file()
    path = tmp_path / "many.gguf"
    path.write_bytes(blob)
    g = GgufFile(str(path))
    names = list(raw)
    shuffled = [names[i] for i in (4, 0, 5, 2, 1, 3)]
    got, released = g.upload_tensors(backend, shuffled)
    page = os.sysconf("SC_PAGESIZE")
    first, last = g.find(names[0]), g.find(names[-1])
    span_end = (last.file_offset + last.n_bytes) // page * page
    span_start = -(-g.data_offset // page) * page
    assert released == span_end - span_start  # everything below the last tensor's end, down to the data section
    for n in shuffled:
        buf, info = got[n]
        assert info.name == n and info.n_bytes == raw[n].nbytes
        assert backend.read(buf, np.uint8, (info.n_bytes,)).tobytes() == raw[n].tobytes()
    again, released2 = g.upload_tensors(backend, names[:2], release_pages=False)  # the released pages re-fault
    assert released2 == 0
    assert backend.read(again[names[1]][0], np.uint8, (raw[names[1]].nbytes,)).tobytes() == raw[names[1]].tobytes()
    from agention_infer_b200 import BackendError
    with pytest.raises(BackendError) as e:
        g.upload_tensors(backend, [names[0], "nope"])
    assert e.value.status == _abi.AGN_ENOTFOUND
    g.close()
