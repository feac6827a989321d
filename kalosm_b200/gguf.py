"""GGUF container: reader (versions 1-3), writer (version 3) and the Llama loader.

Follows fusor-ml/gguf/src/lib.rs:559-613 (`GgufMetadata::read`): magic "GGUF", version, tensor
count, key/value count (lengths are u32 in version 1, u64 later), typed key/values
(lib.rs:346-379), tensor infos (name, dimensions innermost first -- reversed on read so that a
matrix is [N, K] --, ggml type, offset), tensor data from the next multiple of
`general.alignment` (default 32). Strings may carry trailing NUL bytes, which are dropped, and are
decoded leniently (lib.rs:321-334). Tensor names and metadata keys of a Llama checkpoint:
models/kalosm-llama/src/raw/mod.rs:377-415, 473-646.
"""
import struct

import numpy as np

from . import tp

MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", U64: "<Q", I64: "<q", F64: "<d"}


class GgufError(ValueError):
    pass


class _Reader:
    def __init__(self, buf, version=3):
        self.buf, self.pos, self.version = buf, 0, version

    def take(self, n):
        if self.pos + n > len(self.buf):
            raise GgufError("unexpected end of file")
        out = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        return out

    def scalar(self, fmt):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def length(self):
        return self.scalar("<I" if self.version == 1 else "<Q")

    def string(self):
        return self.take(self.length()).rstrip(b"\0").decode("utf-8", errors="replace")

    def value(self, ty):
        if ty in _SCALAR:
            return self.scalar(_SCALAR[ty])
        if ty == BOOL:
            b = self.scalar("<B")
            if b > 1:
                raise GgufError(f"invalid bool value {b}")
            return bool(b)
        if ty == STRING:
            return self.string()
        if ty == ARRAY:
            elem = self.scalar("<I")
            return [self.value(elem) for _ in range(self.length())]
        raise GgufError(f"invalid value type {ty}")


class GgufFile:
    """A parsed GGUF file: `.metadata` {key: value}, `.tensors` {name: (shape, ggml_type, offset)}
    with shape outermost dimension first, `.tensor_data_offset`; tensor bytes are read lazily from a
    memory map."""

    def __init__(self, path):
        self.path = path
        self.data = np.memmap(path, dtype=np.uint8, mode="r")
        r = _Reader(self.data)
        if r.take(4) != MAGIC:
            raise GgufError("not a GGUF file (bad magic)")
        self.version = r.scalar("<I")
        if self.version not in (1, 2, 3):
            raise GgufError(f"unsupported GGUF version {self.version}")
        r.version = self.version
        n_tensors, n_kv = r.length(), r.length()
        self.metadata = {}
        for _ in range(n_kv):
            key = r.string()
            self.metadata[key] = r.value(r.scalar("<I"))
        self.tensors = {}
        for _ in range(n_tensors):
            name = r.string()
            dims = [r.length() for _ in range(r.scalar("<I"))]
            ty = r.scalar("<I")
            self.tensors[name] = (tuple(reversed(dims)), ty, r.scalar("<Q"))
        align = self.metadata.get("general.alignment", DEFAULT_ALIGNMENT)
        if not isinstance(align, int) or isinstance(align, bool) or align <= 0:
            align = DEFAULT_ALIGNMENT
        self.alignment = align
        self.tensor_data_offset = (r.pos + align - 1) // align * align

    def tensor_nbytes(self, name):
        shape, ty, _ = self.tensors[name]
        if ty not in tp.BLOCK:
            raise GgufError(f"tensor {name}: unsupported ggml type {ty}")
        bs, bb = tp.BLOCK[ty]
        n = int(np.prod(shape, dtype=np.int64))
        if shape[-1] % bs:
            raise GgufError(f"tensor {name}: innermost size {shape[-1]} is not a multiple of the block size {bs}")
        return n // bs * bb

    def tensor_bytes(self, name):
        """Raw bytes of a tensor (a view of the memory map)."""
        if name not in self.tensors:
            raise KeyError(name)
        start = self.tensor_data_offset + self.tensors[name][2]
        end = start + self.tensor_nbytes(name)
        if end > len(self.data):
            raise GgufError(f"tensor {name} runs past the end of the file")
        return self.data[start:end]


def _write_value(out, ty, v):
    if ty in _SCALAR:
        out += struct.pack(_SCALAR[ty], v)
    elif ty == BOOL:
        out += struct.pack("<B", 1 if v else 0)
    elif ty == STRING:
        b = v.encode("utf-8")
        out += struct.pack("<Q", len(b)) + b
    elif ty == ARRAY:
        elem, items = v
        out += struct.pack("<IQ", elem, len(items))
        for it in items:
            _write_value(out, elem, it)
    else:
        raise GgufError(f"invalid value type {ty}")


def write_gguf(path, metadata, tensors, alignment=None):
    """Writes a version-3 file. metadata: {key: (value_type, value)} (arrays: (ARRAY, (elem_type,
    items))); tensors: [(name, shape outermost first, ggml_type, bytes-like)]."""
    align = alignment or DEFAULT_ALIGNMENT
    metadata = dict(metadata)
    if alignment:
        metadata["general.alignment"] = (U32, alignment)
    out = bytearray(MAGIC + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for key, (ty, v) in metadata.items():
        _write_value(out, STRING, key)
        out += struct.pack("<I", ty)
        _write_value(out, ty, v)
    offset, blobs = 0, []
    for name, shape, ty, raw in tensors:
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        _write_value(out, STRING, name)
        out += struct.pack("<I", len(shape))
        for d in reversed(shape):
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", ty, offset)
        blobs.append((offset, raw))
        offset = (offset + raw.size + align - 1) // align * align
    out += b"\0" * ((len(out) + align - 1) // align * align - len(out))
    base = len(out)
    with open(path, "wb") as f:
        f.write(out)
        for off, raw in blobs:
            f.write(b"\0" * (base + off - f.tell()))
            f.write(raw.tobytes())


DEFAULT_ROPE_FREQUENCY = 1_000_000.0  # raw/mod.rs:104, used when .rope.freq_base is absent (:385-388)
LAYER_TENSORS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down", "attn_norm", "ffn_norm")


def llama_config(g):
    """Model sizes from the metadata, as Model::from_var_source reads them (raw/mod.rs:377-415)."""
    md = g.metadata
    arch = md.get("general.architecture")
    if not isinstance(arch, str):
        raise GgufError("general.architecture is missing")
    if arch != "llama":
        # qwen2 (half-split RoPE, biases), gemma (sliding windows, q/k norms), phi (fused qkv) are read
        # by the reference (raw/mod.rs:488-646) but not built here: refuse instead of mis-running them
        raise GgufError(f"architecture {arch!r} is not supported (only 'llama')")

    def get(key, default=None):
        v = md.get(arch + key, default)
        if v is None:
            raise GgufError(f"metadata key {arch}{key} is missing")
        return v
    heads, hidden = int(get(".attention.head_count")), int(get(".embedding_length"))
    if "token_embd.weight" not in g.tensors:
        raise GgufError("token_embd.weight is missing")
    return dict(n_layer=int(get(".block_count")), hidden=hidden, ffn=int(get(".feed_forward_length")),
                n_head=heads, n_kv_head=int(get(".attention.head_count_kv")),
                head_dim=int(get(".attention.key_length", hidden // heads)),
                vocab=int(g.tensors["token_embd.weight"][0][0]), ctx=int(get(".context_length")),
                rms_eps=float(get(".attention.layer_norm_rms_epsilon")),
                rope_theta=float(get(".rope.freq_base", DEFAULT_ROPE_FREQUENCY)))


def load_llama(device, path, max_seq_len=None, max_batch=1, comm=None, rope_scaling=None):
    """Builds a `kalosm_b200.Llama` from a GGUF checkpoint (tensor names of raw/mod.rs:473-646;
    a missing output.weight ties the head to the embedding, :480-486). With `comm` every rank loads
    its shard (kalosm_b200.tp). `rope_scaling` = (factor, low_freq_factor, high_freq_factor,
    original_context) is an argument here as it is of Model::from_var_source (raw/mod.rs:271; the
    reference does not read it from the file either); a `rope_freqs.weight` tensor in the file is
    multiplied into the inverse frequencies (raw/mod.rs:417-421, rope.rs:40-49). Metadata keys
    `<arch>.rope.scaling.*` are refused rather than ignored: they ask for a scaling this loader
    would otherwise silently drop."""
    from . import F32 as F32_TYPE, Llama
    g = GgufFile(path)
    c = llama_config(g)
    rank, size = (comm.rank, comm.size) if comm is not None else (0, 1)
    scaling_keys = [k for k in g.metadata if ".rope.scaling." in k]
    if scaling_keys and rope_scaling is None:
        raise GgufError(f"the file asks for RoPE scaling ({', '.join(sorted(scaling_keys))}); pass rope_scaling=")
    if size > 1 and "output.weight" not in g.tensors:
        raise GgufError("a tensor-parallel model needs output.weight (tied embeddings are not sharded)")
    m = Llama(device, n_layer=c["n_layer"], hidden=c["hidden"], ffn=c["ffn"], n_head=c["n_head"],
              n_kv_head=c["n_kv_head"], head_dim=c["head_dim"], vocab=c["vocab"],
              max_seq_len=max_seq_len or c["ctx"], max_batch=max_batch, rms_eps=c["rms_eps"],
              rope_theta=c["rope_theta"], rope_scaling=rope_scaling, comm=comm)
    if "rope_freqs.weight" in g.tensors:
        shape, ty, _ = g.tensors["rope_freqs.weight"]
        if ty != F32_TYPE or int(np.prod(shape)) != c["head_dim"] // 2:
            raise GgufError("rope_freqs.weight must be head_dim / 2 f32 values")
        m.set_rope_freqs(np.frombuffer(bytes(g.tensor_bytes("rope_freqs.weight")), dtype=np.float32))

    def put(short, layer, name):
        shape, ty, _ = g.tensors[name]
        raw = g.tensor_bytes(name)
        if short.endswith("_norm"):
            if ty != F32_TYPE:
                raise GgufError(f"{name}: norm weights must be f32")
            m.set_tensor(short, layer, ty, shape, np.array(raw))
            return
        part, part_shape = tp.shard(short, raw, ty, shape, rank, size)
        m.set_tensor(short, layer, ty, part_shape, part)
    put("token_embd", -1, "token_embd.weight")
    put("output_norm", -1, "output_norm.weight")
    if "output.weight" in g.tensors:
        put("output", -1, "output.weight")
    for i in range(c["n_layer"]):
        for short in LAYER_TENSORS:
            name = f"blk.{i}.{short}.weight"
            if name not in g.tensors:
                raise GgufError(f"{name} is missing")
            put(short, i, name)
    return m
