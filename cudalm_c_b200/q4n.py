"""Exact 4-bit export of a parameter vector and the quantised container file.

Mirrors the reference's `quantize <in> <out> q4n` command and its loader (quantize_params / dequantize_params with
qtype 3, cudalm.cu:639-656, 688-695; TLQ1 / TLQ2 container, 9783-9793, 438-450).  The scale search, the nibble
packing and the decode run on the device (qlmb_q4n_export / qlmb_q4n_decode); only the walk that finds where each
group of a stream starts is host work, because a group's position depends on the kind of every group before it.
"""
import ctypes as C

import numpy as np
import torch

from ._lib import check, lib, ptr, stream_ptr

GROUP = 128          # the reference's group for q4n
QTYPE = 3


def export(P, group=GROUP):
    """P: fp32 CUDA vector -> (stream as a uint8 CUDA tensor, number of groups stored raw)"""
    assert P.is_cuda and P.dtype == torch.float32 and P.is_contiguous()
    L = lib()
    n = P.numel()
    cap = int(L.qlmb_q4n_max_bytes(n, group))
    out = torch.empty(cap, dtype=torch.uint8, device=P.device)
    work = torch.empty((int(L.qlmb_q4n_work_bytes(n, group)) + 7) // 8, dtype=torch.int64, device=P.device)
    totals = torch.zeros(2, dtype=torch.int64, device=P.device)
    check(L.qlmb_q4n_export(ptr(out), cap, ptr(totals), ptr(P), n, group, ptr(work), stream_ptr()))
    length, raw = (int(v) for v in totals.cpu())
    assert length <= cap
    return out[:length], raw


def index(stream_host, n, group=GROUP):
    """byte offset of every group of a host stream (numpy uint8); the last entry is the stream's length"""
    ng = (n + group - 1) // group
    off = np.zeros(ng + 1, np.uint64)
    check(lib().qlmb_q4n_index(stream_host.ctypes.data_as(C.c_void_p), stream_host.size, n, group, off.ctypes.data_as(C.c_void_p)))
    return off


def decode(stream_host, n, device, group=GROUP, off=None):
    """host stream (numpy uint8) -> fp32 CUDA vector of n values, decoded on the device"""
    off = index(stream_host, n, group) if off is None else off
    body = torch.from_numpy(stream_host[:int(off[-1])].copy()).to(device)
    offd = torch.from_numpy(off.view(np.int64)).to(device)
    P = torch.empty(n, dtype=torch.float32, device=device)
    check(lib().qlmb_q4n_decode(ptr(P), ptr(body), ptr(offd), n, group, stream_ptr()))
    return P


def save(path, hdr13, P, tok_blob=b"", group=GROUP):
    """Writes the TLQ1 / TLQ2 file of a parameter vector on the device; returns (body bytes, raw groups)."""
    q, raw = export(P, group)
    qh = q.cpu().numpy()
    hdr = np.ascontiguousarray(hdr13, np.int32)
    assert hdr.size == 13
    blob = np.frombuffer(tok_blob, np.uint8) if tok_blob else None
    check(lib().qlmb_qfile_write(str(path).encode(), hdr.ctypes.data_as(C.c_void_p), QTYPE, group, qh.ctypes.data_as(C.c_void_p),
                                 qh.size, None if blob is None else blob.ctypes.data_as(C.c_void_p), 0 if blob is None else blob.size))
    return qh.size, raw


def read(path):
    """-> (hdr13, qtype, group, the bytes after the header as numpy uint8: body, then the tokenizer trailer)"""
    hdr = np.zeros(13, np.int32)
    qtype, group, rest = C.c_int(0), C.c_int(0), C.c_ulonglong(0)
    L = lib()
    check(L.qlmb_qfile_read_header(str(path).encode(), hdr.ctypes.data_as(C.c_void_p), C.byref(qtype), C.byref(group), C.byref(rest)))
    buf = np.zeros(rest.value, np.uint8)
    check(L.qlmb_qfile_read(str(path).encode(), buf.ctypes.data_as(C.c_void_p), rest.value))
    return hdr, qtype.value, group.value, buf


def load(path, n, device):
    """Reads a q4n TLQ file of n parameters: (hdr13, fp32 CUDA vector, tokenizer blob bytes)."""
    hdr, qtype, group, buf = read(path)
    if qtype != QTYPE:
        raise ValueError("%s: quantisation type %d, only q4n (3) is read here" % (path, qtype))
    off = index(buf, n, group)
    end = int(off[-1])
    tl = int(np.frombuffer(buf[end:end + 4].tobytes(), np.int32)[0]) if end + 4 <= buf.size else 0
    blob = buf[end + 4:end + 4 + tl].tobytes() if tl > 0 and end + 4 + tl <= buf.size else b""
    return hdr, decode(buf, n, device, group, off), blob
