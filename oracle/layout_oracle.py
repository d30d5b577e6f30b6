"""CPU restatement of the network parameter layout conversion (TEST INFRASTRUCTURE ONLY).

Follows the golden model the reference's own unit test builds
(tools/gfx-unit-test/neural-slang-network-converter.cpp:76-126 for the CUDA tile order and offsets,
:128-196 for the element counts and the expected arrays):
  logical  = per layer in*out weights, row-major [out][in], then out biases if the layer has one
  physical = per layer align16(in)*align16(out) weights in 16x16 tiles, tile (input tile, output tile) at
             (input_tile * tile_cols + output_tile) * 256 with tile_cols = align16(out)/16, inside a
             tile the tensor-core B-fragment register order, then align16(out) bias slots (reserved
             also for layers without a bias); padding is zero.
"""
import numpy as np


def align16(v):
    return (v + 15) // 16 * 16


def native_tile_pos(row, col):
    """Position of (row = input in tile, col = output in tile) inside the 256-element tile."""
    row_group, row_in_group = divmod(row, 8)
    tid_local, pair = divmod(row_in_group, 2)
    sub, gid = divmod(col, 8)
    lane = gid * 4 + tid_local
    return lane * 8 + sub * 4 + row_group * 2 + pair


def sizes(dims, bias_mask):
    logical = physical = 0
    for l in range(len(dims) - 1):
        i, o = dims[l], dims[l + 1]
        logical += i * o + (o if (bias_mask >> l) & 1 else 0)
        physical += align16(i) * align16(o) + align16(o)
    return logical, physical


def to_optimal(portable, dims, bias_mask):
    logical, physical = sizes(dims, bias_mask)
    assert portable.size == logical
    out = np.zeros(physical, dtype=portable.dtype)
    lo = po = 0
    for l in range(len(dims) - 1):
        i, o = dims[l], dims[l + 1]
        tile_cols = align16(o) // 16
        for oi in range(o):
            for ii in range(i):
                tile_base = ((ii // 16) * tile_cols + oi // 16) * 256
                out[po + tile_base + native_tile_pos(ii % 16, oi % 16)] = portable[lo + oi * i + ii]
            if (bias_mask >> l) & 1:
                out[po + align16(i) * align16(o) + oi] = portable[lo + i * o + oi]
        lo += i * o + (o if (bias_mask >> l) & 1 else 0)
        po += align16(i) * align16(o) + align16(o)
    return out


def reference_test_values(n):
    """makePortableValue of the reference's unit test (:149-153)."""
    idx = np.arange(n)
    return (((idx * 37 + 19) % 257) - 128).astype(np.float32) * 0.125


# ---- cooperative-vector matrix layouts ------------------------------------------------------------
ROW_MAJOR, COLUMN_MAJOR, INFERENCING_OPTIMAL, TRAINING_OPTIMAL = 0, 1, 2, 3


def matrix_size(rows, cols, elem_size, layout, stride=0):
    """Bytes a rows x cols matrix takes: packed or strided row-/column-major; the optimal layouts pad both
    extents to multiples of 16 (16x16 tiles)."""
    if layout == ROW_MAJOR:
        return (rows - 1) * stride + cols * elem_size if stride else rows * cols * elem_size
    if layout == COLUMN_MAJOR:
        return (cols - 1) * stride + rows * elem_size if stride else rows * cols * elem_size
    return -(-rows // 16) * 16 * (-(-cols // 16) * 16) * elem_size


def matrix_to_bytes(m, np_dtype, layout, stride=0, fill=0):
    """The bytes of matrix m (2-D float array) in the given layout and element type; bytes that the layout
    does not define (stride gaps) hold `fill`."""
    import numpy as np
    rows, cols = m.shape
    es = np.dtype(np_dtype).itemsize
    out = np.full(matrix_size(rows, cols, es, layout, stride), fill, dtype=np.uint8)
    vals = m.astype(np_dtype)
    if layout in (ROW_MAJOR, COLUMN_MAJOR):
        v = vals if layout == ROW_MAJOR else vals.T
        st = stride if stride else v.shape[1] * es
        for r in range(v.shape[0]):
            out[r * st: r * st + v.shape[1] * es] = np.ascontiguousarray(v[r]).view(np.uint8)
        return out
    pr, pc = -(-rows // 16) * 16, -(-cols // 16) * 16
    padded = np.zeros((pr, pc), dtype=np_dtype)
    padded[:rows, :cols] = vals
    tiles = padded.reshape(pr // 16, 16, pc // 16, 16).transpose(0, 2, 1, 3)   # [tile row][tile col][r][c]
    return np.ascontiguousarray(tiles).view(np.uint8).reshape(-1).copy()
