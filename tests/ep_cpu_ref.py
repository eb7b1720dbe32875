"""CPU stand-ins for the device side of the expert-parallel exchange (hq_ep_pack / hq_ep_unpack_meta and the local
expert block), restating the slab layout of include/hanzoquant_b200.h byte for byte with numpy.  Test
infrastructure: used by the gloo protocol tests and as the checker of the CUDA pack / unpack kernels."""
import numpy as np
import torch


def cpu_pack(lay, x, ids, weights, send):
    """16-bit wire only (the FP8 wire is checked on the GPU against oracle.formats)."""
    t, k = ids.shape
    buf = send.numpy().reshape(lay.world, lay.rows_per_peer * lay.row_bytes)
    ids_np = ids.numpy().astype(np.int64)
    w_np = weights.numpy().astype(np.float32)
    wire = x.to(torch.bfloat16 if lay.wire_dtype == 2 else torch.float16).contiguous().view(torch.uint8).numpy()
    back_map = np.full((t, lay.world), -1, np.int32)
    meta_off = lay.capacity * lay.row_bytes
    for d in range(lay.world):
        meta = np.zeros((lay.capacity, k, 2), np.int32)
        meta[:, :, 0] = -1
        for tok in range(t):
            mine = (ids_np[tok] >= 0) & (ids_np[tok] // lay.experts_per_rank == d) & \
                   (ids_np[tok] < lay.world * lay.experts_per_rank)
            if mine.any():
                buf[d, tok * lay.row_bytes:(tok + 1) * lay.row_bytes] = wire[tok]
                back_map[tok, d] = d * lay.rows_per_peer + tok
            meta[tok, mine, 0] = ids_np[tok][mine] - d * lay.experts_per_rank
            meta[tok, mine, 1] = w_np[tok][mine].view(np.int32)
        raw = meta.reshape(-1).view(np.uint8)
        buf[d, meta_off:meta_off + raw.size] = raw
    return torch.from_numpy(back_map)


def cpu_unpack(lay, recv):
    buf = recv.numpy().reshape(lay.world, lay.rows_per_peer * lay.row_bytes)
    k = lay.top_k
    ids = np.full((lay.world, lay.rows_per_peer, k), -1, np.int32)
    w = np.zeros((lay.world, lay.rows_per_peer, k), np.float32)
    meta_off = lay.capacity * lay.row_bytes
    for s in range(lay.world):
        meta = buf[s, meta_off:meta_off + lay.capacity * k * 8].copy().view(np.int32).reshape(lay.capacity, k, 2)
        ids[s, :lay.capacity] = meta[:, :, 0]
        w[s, :lay.capacity] = meta[:, :, 1].copy().view(np.float32)
    return torch.from_numpy(ids.reshape(-1, k)), torch.from_numpy(w.reshape(-1, k))


def cpu_rows(lay, recv):
    """Received payload rows as f32 [world * rows_per_peer, hidden] (16-bit wire)."""
    dt = torch.bfloat16 if lay.wire_dtype == 2 else torch.float16
    return recv.view(dt).view(lay.world * lay.rows_per_peer, lay.hidden).to(torch.float32)


def cpu_reduce(y_rows, weights, row_map, out_dtype, addend):
    y = y_rows.to(torch.float32).numpy()
    rm = row_map.numpy().astype(np.int64)
    w = weights.numpy()
    out = np.zeros((rm.shape[0], y.shape[1]), np.float32)
    for s in range(rm.shape[1]):
        ok = rm[:, s] >= 0
        out[ok] += w[ok, s:s + 1] * y[rm[ok, s]]
    if addend is not None:
        out += addend.to(torch.float32).numpy()
    return torch.from_numpy(out).to(out_dtype)
