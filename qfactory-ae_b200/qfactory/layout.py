"""The packed "tile-128 interleaved" layout, in vectorised torch (any device).

Layout (the same one `qfb_pack` in the native library writes; see
include/qfactory_b200.h): rows = output features, padded to a multiple of 128 and cut in
tiles of 128; along K a row is cut in 16-byte vectors (128/bits codes; for 3 bits a unit
of 128 codes = two 2-bit-plane vectors + one 1-bit-plane vector).

    qweight  u8 [tiles][vectors along K][128 rows][16]
    scales   f16[tiles][K/group][128 rows]
    zeros    u8 [tiles][K/group][128 rows]      effective zero min(z+1, 2^b-1)

This replaces the reference's N-major layout (reference: qfactory/convert.py:55-81); the
intra-word field order of the 2/4/8-bit formats is the reference's PERMUTE_ORDER
(qfactory/convert.py:49-53), which is what makes one LOP3 yield an fp16x2 pair.
"""
from __future__ import annotations

import torch

TILE = 128
LAYOUT_TILE, LAYOUT_FRAGMENT = 0, 1  # QFB_LAYOUT_* of the C ABI


def unit_k(bits: int) -> int:
    return {8: 16, 4: 32, 2: 64, 3: 128}[bits]


def unit_vecs(bits: int) -> int:
    return 3 if bits == 3 else 1


def padded_rows(n: int) -> int:
    return (n + TILE - 1) // TILE * TILE


def check_shape(N: int, K: int, bits: int, GS: int) -> None:
    if bits not in (2, 3, 4, 8):
        raise ValueError(f"unsupported bit width {bits}")
    assert K % 64 == 0 and K % unit_k(bits) == 0, f"K={K} must be a multiple of 64 and of {unit_k(bits)}"
    if GS != -1:
        assert GS > 0 and GS % 64 == 0 and K % GS == 0 and GS % unit_k(bits) == 0, \
            f"group size {GS} must be a multiple of 64 (128 for 3-bit) dividing K={K}"


def field_elements(bits: int) -> list[int]:
    """Element held by field f of a 32-bit word (pair interleave for 2/4-bit)."""
    pf = 32 // bits
    if bits == 8:
        return list(range(pf))
    return list(range(0, pf, 2)) + list(range(1, pf, 2))


def plane1_bit(e: int) -> int:
    """Bit of element e (0..31) in a word of the 3-bit format's 1-bit plane."""
    h, el = e >> 4, e & 15
    f, parity = el >> 1, el & 1
    base = (0, 1, 8, 9)[2 * h + (f >> 2)]
    return base + 2 * (f & 3) + 16 * parity


def _words_to_bytes(words: torch.Tensor) -> torch.Tensor:
    sh = torch.arange(4, device=words.device, dtype=torch.int64) * 8
    return ((words.unsqueeze(-1) >> sh) & 0xFF).to(torch.uint8)


def _bytes_to_words(b: torch.Tensor) -> torch.Tensor:
    sh = torch.arange(4, device=b.device, dtype=torch.int64) * 8
    return (b.to(torch.int64) << sh).sum(-1)


def _pack_fields(v: torch.Tensor, bits: int) -> torch.Tensor:
    """v int64 [..., 32/bits] elements of one word in K order -> int64 words [...]."""
    order = torch.tensor(field_elements(bits), device=v.device)
    sh = torch.arange(32 // bits, device=v.device, dtype=torch.int64) * bits
    return (v[..., order] << sh).sum(-1)


def _unpack_fields(words: torch.Tensor, bits: int) -> torch.Tensor:
    pf = 32 // bits
    sh = torch.arange(pf, device=words.device, dtype=torch.int64) * bits
    fields = (words.unsqueeze(-1) >> sh) & ((1 << bits) - 1)
    out = torch.empty_like(fields)
    out[..., torch.tensor(field_elements(bits), device=words.device)] = fields
    return out


def _rows_per_batch(K: int) -> int:
    return max(TILE, (1 << 24) // K // TILE * TILE)


def pack_weight(q: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 codes [K, N] -> int8 [Npad, K*bits/8] (flat tile-128 layout)."""
    K, N = q.shape
    Np = padded_rows(N)
    uk, nv = unit_k(bits), unit_vecs(bits)
    units = K // uk
    out = torch.empty(Np // TILE, units * nv, TILE, 16, dtype=torch.uint8, device=q.device)
    step = _rows_per_batch(K)
    for r0 in range(0, Np, step):
        r1 = min(Np, r0 + step)
        blk = torch.zeros(r1 - r0, K, dtype=torch.int64, device=q.device)
        n1 = min(r1, N)
        if n1 > r0:
            blk[: n1 - r0] = q[:, r0:n1].t()
        T = (r1 - r0) // TILE
        if bits != 3:
            words = _pack_fields(blk.view(T, TILE, units, 4, 32 // bits), bits)  # [T,128,units,4]
            by = _words_to_bytes(words).view(T, TILE, units, 16)
            out[r0 // TILE : r1 // TILE] = by.permute(0, 2, 1, 3)
        else:
            lo = _pack_fields((blk & 3).view(T, TILE, units, 2, 4, 16), 2)  # [T,128,units,2,4]
            pos = torch.tensor([plane1_bit(e) for e in range(32)], device=q.device, dtype=torch.int64)
            hi = ((((blk >> 2) & 1).view(T, TILE, units, 4, 32)) << pos).sum(-1)  # [T,128,units,4]
            by = torch.cat([_words_to_bytes(lo).view(T, TILE, units, 2, 16),
                            _words_to_bytes(hi).view(T, TILE, units, 1, 16)], dim=3)  # [T,128,units,3,16]
            out[r0 // TILE : r1 // TILE] = by.permute(0, 2, 3, 1, 4).reshape(T, units * 3, TILE, 16)
    return out.view(Np, K * bits // 8).view(torch.int8)


def unpack_weight(w: torch.Tensor, N: int, K: int, bits: int) -> torch.Tensor:
    """Inverse of pack_weight: int8 [Npad, K*bits/8] -> int32 codes [K, N]."""
    Np = padded_rows(N)
    uk, nv = unit_k(bits), unit_vecs(bits)
    units = K // uk
    T = Np // TILE
    b = w.contiguous().view(torch.uint8).view(T, units, nv, TILE, 16)
    if bits != 3:
        words = _bytes_to_words(b.view(T, units, TILE, 4, 4))
        q = _unpack_fields(words, bits)  # [T,units,128,4,pf]
        q = q.permute(0, 2, 1, 3, 4).reshape(Np, K)
    else:
        lo = _unpack_fields(_bytes_to_words(b[:, :, :2].reshape(T, units, 2, TILE, 4, 4)), 2)  # [T,u,2,128,4,16]
        lo = lo.permute(0, 3, 1, 2, 4, 5).reshape(Np, K)
        hw = _bytes_to_words(b[:, :, 2].reshape(T, units, TILE, 4, 4))  # [T,u,128,4]
        pos = torch.tensor([plane1_bit(e) for e in range(32)], device=w.device, dtype=torch.int64)
        hi = ((hw.unsqueeze(-1) >> pos) & 1).permute(0, 2, 1, 3, 4).reshape(Np, K)
        q = lo | (hi << 2)
    return q[:N].t().contiguous().to(torch.int32)


def _tile_major(a: torch.Tensor, N: int) -> torch.Tensor:
    """[G, N] -> [tiles, G, 128] with zero padding of the rows."""
    G = a.shape[0]
    Np = padded_rows(N)
    buf = torch.zeros(Np, G, dtype=a.dtype, device=a.device)
    buf[:N] = a.t()
    return buf.view(Np // TILE, TILE, G).permute(0, 2, 1).contiguous()


def pack_scale(s: torch.Tensor) -> torch.Tensor:
    """fp16 [G, N] -> fp16 [Npad, G] (flat [tiles][G][128])."""
    G, N = s.shape
    return _tile_major(s, N).view(padded_rows(N), G)


def effective_zero(z: torch.Tensor, bits: int) -> torch.Tensor:
    """GPTQ-convention zero -> the value the kernel subtracts: min(z+1, 2^b-1)
    (reference: qfactory/convert.py:76)."""
    return (z + 1).clamp(max=(1 << bits) - 1)


def pack_zero(z: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 GPTQ zeros [G, N] -> int8 [Npad, G] holding the effective zero per byte."""
    G, N = z.shape
    ze = effective_zero(z, bits).to(torch.uint8)
    return _tile_major(ze, N).view(padded_rows(N), G).view(torch.int8)


def unpack_scale(s: torch.Tensor, N: int) -> torch.Tensor:
    """fp16 [Npad, G] packed -> fp16 [G, N]."""
    Np, G = s.shape
    return s.contiguous().view(Np // TILE, G, TILE).permute(1, 0, 2).reshape(G, Np)[:, :N].contiguous()


def unpack_zero(z: torch.Tensor, N: int) -> torch.Tensor:
    """int8 [Npad, G] packed -> effective zeros int32 [G, N]."""
    Np, G = z.shape
    zz = z.contiguous().view(torch.uint8).view(Np // TILE, G, TILE).permute(1, 0, 2).reshape(G, Np)
    return zz[:, :N].to(torch.int32).contiguous()


# ---------------------------------------------------------------------------------------
# Fragment layouts (K % 128 == 0): the same codes permuted so that the words a lane
# holds are the A fragments a thread feeds to mma.sync.m16n8k16 (include/qfactory_b200.h and
# csrc/qfb_common.cuh).  Lane (g = lane // 4, t = lane % 4) of the 64-row half wt of a tile owns,
# for each of its four row blocks rb, rows g and g + 8 (h = 0, 1) at k = 16*ks + 4*t + kk:
#   word of the lane that holds code (rb, h, kk):  4-bit rb | 8-bit 2*rb + h | 2-bit rb // 2
#   bit position inside that word:                 frag_bit_of below
#   (3-bit: three words per lane, placed bit by bit: frag_code_bit below)
#   qweight  [tiles][2][K/16] steps of 128*bits bytes: lane-major words (8-bit: two 512-byte chunks,
#            row blocks 0,1 then 2,3)
#   scales / zeros  [tiles][K/group][128], position wt*64 + g*8 + rb*2 + h <-> row wt*64 + rb*16 + h*8 + g
# ---------------------------------------------------------------------------------------
NIBBLE_K = [(i >> 2) + 2 * ((i >> 1) & 1) for i in range(8)]  # 4-bit: k offset held by nibble i (row = i & 1)


def frag_word_of(bits: int, rb: int, h: int) -> int:
    return rb if bits == 4 else (2 * rb + h if bits == 8 else rb // 2)


def frag_bit_of(bits: int, rb: int, h: int, kk: int) -> int:
    if bits == 8:
        return 8 * kk
    if bits == 4:
        return 4 * ((kk >> 1) * 2 + (kk & 1) * 4 + h)
    return (rb & 1) * 4 + h * 2 + (kk & 1) * 16 + (kk >> 1) * 8


def frag_code_bit(bits: int, rb: int, h: int, kk: int, b: int):
    """(word of the lane, bit inside it) that holds bit b of code (rb, h, kk).  2-, 4- and 8-bit codes
    are contiguous fields.  3-bit: three words per lane; a half-word holds five fields (offsets 0, 3,
    6, 9, 12) and a spare bit; row blocks 0..2 live in word rb (rows g at offsets 0 / 9, rows g + 8 at
    3 / 12 for k 4t.. / 4t+2..), row block 3 at offset 6 of words 0, 1 (rows g) and 2 (rows g + 8,
    k 4t..) and, for rows g + 8, k 4t+2.., in the spare bits: bit b of the code is bit 15 (31) of word b."""
    if bits != 3:
        return frag_word_of(bits, rb, h), frag_bit_of(bits, rb, h, kk) + b
    half, khi = (kk & 1) * 16, kk >> 1
    if rb < 3:
        return rb, half + h * 3 + khi * 9 + b
    if h == 1 and khi == 1:
        return b, half + 15
    return (2 if h == 1 else khi), half + 6 + b


def frag_word_slot(bits: int, lane: int, j: int) -> int:
    """Index (in 32-bit words) of word j of a lane inside a k-step."""
    if bits == 8:
        return (j >> 2) * 128 + lane * 4 + (j & 3)
    if bits == 3:
        return j * 32 + lane
    return lane * bits + j


def fragment_supported(N: int, K: int, bits: int, GS: int) -> bool:
    if bits == 3:
        return K % 128 == 0 and (GS == -1 or GS % 128 == 0)
    return bits in (2, 4, 8) and K % 128 == 0 and (GS in (-1, 64) or GS % 128 == 0)


def resolve_layout(layout, N: int, K: int, bits: int, GS: int, batch_size: int = 1) -> int:
    """'tile' | 'fragment' | 'auto' | 0 | 1 | None -> LAYOUT_*.  'auto' (and None) picks the fragment
    layout whenever the shape allows it (K % 128 == 0, group 64 or a multiple of 128): it
    feeds the fastest kernel up to 16 rows and the tcgen05 kernel within a few percent of the tile
    layout above.  `batch_size` is accepted for the callers' convenience and does not matter."""
    if layout in (LAYOUT_TILE, "tile"):
        return LAYOUT_TILE
    if layout in (LAYOUT_FRAGMENT, "fragment"):
        assert fragment_supported(N, K, bits, GS), "the fragment layout needs K % 128 == 0 and groups of 64 (not 3-bit) or multiples of 128"
        return LAYOUT_FRAGMENT
    assert layout in (None, "auto"), f"unknown layout {layout!r}"
    return LAYOUT_FRAGMENT if fragment_supported(N, K, bits, GS) else LAYOUT_TILE


def frag_row_of_pos(device=None) -> torch.Tensor:
    pos = torch.arange(TILE, device=device)
    return (pos >> 6) * 64 + ((pos >> 1) & 3) * 16 + (pos & 1) * 8 + ((pos >> 3) & 7)


def _frag_slots(bits: int, device):
    """For every (rb, h, g, t, kk) and code bit b: word slot inside the k-step and bit position."""
    slot = torch.empty(4, 2, 8, 4, 4, bits, dtype=torch.int64)
    bit = torch.empty(4, 2, 8, 4, 4, bits, dtype=torch.int64)
    for rb in range(4):
        for h in range(2):
            for g in range(8):
                for t in range(4):
                    for kk in range(4):
                        for b in range(bits):
                            wj, pos = frag_code_bit(bits, rb, h, kk, b)
                            slot[rb, h, g, t, kk, b] = frag_word_slot(bits, g * 4 + t, wj)
                            bit[rb, h, g, t, kk, b] = pos
    return slot.to(device), bit.to(device)


def pack_weight_fragment(q: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """int32 codes [K, N] -> int8 [Npad, K*bits/8] in fragment order."""
    K, N = q.shape
    Np = padded_rows(N)
    T = Np // TILE
    blk = torch.zeros(Np, K, dtype=torch.int64, device=q.device)
    blk[:N] = q.t()
    v = blk.view(T, 2, 4, 2, 8, K // 16, 4, 4).permute(0, 1, 5, 2, 3, 4, 6, 7)   # [tile, wt, ks, rb, h, g, t, kk]
    slot, bit = _frag_slots(bits, q.device)
    words = torch.zeros(T, 2, K // 16, 32 * bits, dtype=torch.int64, device=q.device)
    planes = torch.arange(bits, device=q.device)
    vbits = ((v.unsqueeze(-1) >> planes) & 1) << bit                                 # every code bit at its place
    words.scatter_add_(3, slot.flatten().expand(T, 2, K // 16, -1), vbits.reshape(T, 2, K // 16, -1))
    return _words_to_bytes(words).reshape(Np, K * bits // 8).view(torch.int8)


def unpack_weight_fragment(w: torch.Tensor, N: int, K: int, bits: int = 4) -> torch.Tensor:
    Np = padded_rows(N)
    T = Np // TILE
    words = _bytes_to_words(w.contiguous().view(torch.uint8).view(T, 2, K // 16, 32 * bits, 4))
    slot, bit = _frag_slots(bits, w.device)
    vb = (words[..., slot.flatten()] >> bit.flatten()) & 1                           # [tile, wt, ks, rb*h*g*t*kk*b]
    v = (vb.view(T, 2, K // 16, -1, bits) << torch.arange(bits, device=w.device)).sum(-1)
    v = v.view(T, 2, K // 16, 4, 2, 8, 4, 4).permute(0, 1, 3, 4, 5, 2, 6, 7)        # [tile, wt, rb, h, g, ks, t, kk]
    return v.reshape(Np, K)[:N].t().contiguous().to(torch.int32)


def _to_fragment_rows(a: torch.Tensor) -> torch.Tensor:
    """[Npad, G] flat tile-major -> the same with the 128 rows of every tile in fragment order."""
    Np, G = a.shape
    return a.contiguous().view(Np // TILE, G, TILE)[:, :, frag_row_of_pos(a.device)].contiguous().view(Np, G)


def _from_fragment_rows(a: torch.Tensor) -> torch.Tensor:
    Np, G = a.shape
    out = torch.empty_like(a.contiguous().view(Np // TILE, G, TILE))
    out[:, :, frag_row_of_pos(a.device)] = a.contiguous().view(Np // TILE, G, TILE)
    return out.view(Np, G)


def pack_scale_fragment(s: torch.Tensor) -> torch.Tensor:
    return _to_fragment_rows(pack_scale(s))


def pack_zero_fragment(z: torch.Tensor, bits: int) -> torch.Tensor:
    return _to_fragment_rows(pack_zero(z, bits))


def unpack_scale_fragment(s: torch.Tensor, N: int) -> torch.Tensor:
    return unpack_scale(_from_fragment_rows(s), N)


def unpack_zero_fragment(z: torch.Tensor, N: int) -> torch.Tensor:
    return unpack_zero(_from_fragment_rows(z), N)
