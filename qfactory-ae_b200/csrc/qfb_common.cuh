// Shared device helpers: packed-layout geometry, streaming loads and the in-register
// code extraction (LOP3 / PRMT magic-number trick) used by every kernel of the library.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qfactory_b200.h"

namespace qfb {

constexpr int kTileRows = 128;  // rows (output features) per packed tile

// ---------------------------------------------------------------------------
// Geometry of the packed layout per bit width.  A "unit" is the smallest run of
// codes along K one row decodes at a time: one 16-byte vector for 2/4/8 bits,
// three vectors (two 2-bit-plane chunks + one 1-bit-plane chunk) for 3 bits.
// ---------------------------------------------------------------------------
template <int BITS> struct Geo;
template <> struct Geo<8> { static constexpr int kUnitK = 16, kUnitVecs = 1; };
template <> struct Geo<4> { static constexpr int kUnitK = 32, kUnitVecs = 1; };
template <> struct Geo<2> { static constexpr int kUnitK = 64, kUnitVecs = 1; };
template <> struct Geo<3> { static constexpr int kUnitK = 128, kUnitVecs = 3; };

__host__ __device__ inline int unit_k(int bits) { return bits == 8 ? 16 : bits == 4 ? 32 : bits == 2 ? 64 : 128; }
__host__ __device__ inline int unit_vecs(int bits) { return bits == 3 ? 3 : 1; }
__host__ __device__ inline int padded_rows(int n) { return (n + kTileRows - 1) / kTileRows * kTileRows; }

// ---------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// (a & b) | c
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// a | (b & c)
__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xF8;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Programmatic dependent launch: both are no-ops when the grid was launched without
// the programmatic-stream-serialisation attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Code extraction.  Every decoder produces fp16x2 pairs holding (q - z) EXACTLY:
// a field is OR-ed into the mantissa of a power-of-two "magic" half whose unit in
// the last place lines up with the field's bit offset, giving magic + q, and the
// zero-point is subtracted as magic + z.  Both are exactly representable, so the
// difference is exact (this is the reference's own trick, qfactory/include/utils.h:
// 11-25,46-62, extended to un-shifted fields at several bit offsets).
//
// zmagic(z) builds the per-group subtrahends; decode8(...) hands the caller four
// fp16x2 values = eight consecutive codes along K.
// ---------------------------------------------------------------------------
template <int BITS> struct Codec;

template <> struct Codec<4> {
  struct ZM { uint32_t lo, hi; };
  __device__ static __forceinline__ ZM zmagic(uint32_t z) {
    uint32_t zz = z * 0x00010001u;
    return {0x64006400u | zz, 0x54005400u | (zz << 4)};
  }
  // word -> 8 codes (4 pairs).  nibble p of the word holds element (p<4 ? 2p : 2(p-4)+1).
  __device__ static __forceinline__ void word(uint32_t w, const ZM& zm, __half2 (&d)[4]) {
    uint32_t t = w >> 8;
    d[0] = __hsub2(as_h2(lop3_and_or(w, 0x000f000fu, 0x64006400u)), as_h2(zm.lo));
    d[1] = __hsub2(as_h2(lop3_and_or(w, 0x00f000f0u, 0x54005400u)), as_h2(zm.hi));
    d[2] = __hsub2(as_h2(lop3_and_or(t, 0x000f000fu, 0x64006400u)), as_h2(zm.lo));
    d[3] = __hsub2(as_h2(lop3_and_or(t, 0x00f000f0u, 0x54005400u)), as_h2(zm.hi));
  }
  // f(j8, d[4]) for each group of 8 codes of the unit, in K order
  template <class F> __device__ static __forceinline__ void unit(const uint4* v, const ZM& zm, F&& f) {
    const uint32_t w[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 d[4];
      word(w[j], zm, d);
      f(j, d);
    }
  }
};

template <> struct Codec<8> {
  struct ZM { uint32_t m; };
  __device__ static __forceinline__ ZM zmagic(uint32_t z) { return {0x64006400u | (z * 0x00010001u)}; }
  template <class F> __device__ static __forceinline__ void unit(const uint4* v, const ZM& zm, F&& f) {
    const uint32_t w[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      __half2 d[4];
      d[0] = __hsub2(as_h2(prmt(w[2 * j], 0x64646464u, 0x4140u)), as_h2(zm.m));
      d[1] = __hsub2(as_h2(prmt(w[2 * j], 0x64646464u, 0x4342u)), as_h2(zm.m));
      d[2] = __hsub2(as_h2(prmt(w[2 * j + 1], 0x64646464u, 0x4140u)), as_h2(zm.m));
      d[3] = __hsub2(as_h2(prmt(w[2 * j + 1], 0x64646464u, 0x4342u)), as_h2(zm.m));
      f(j, d);
    }
  }
};

template <> struct Codec<2> {
  struct ZM { uint32_t m[4]; };
  __device__ static __forceinline__ ZM zmagic(uint32_t z) {
    uint32_t zz = z * 0x00010001u;
    return {{0x64006400u | zz, 0x5C005C00u | (zz << 2), 0x54005400u | (zz << 4), 0x4C004C00u | (zz << 6)}};
  }
  // 2-bit field f (bit offset 2f, f < 8) holds element 2f, the field 16 bits above it 2f+1
  __device__ static __forceinline__ void half_word(uint32_t w, const ZM& zm, __half2 (&d)[4]) {
    d[0] = __hsub2(as_h2(lop3_and_or(w, 0x00030003u, 0x64006400u)), as_h2(zm.m[0]));
    d[1] = __hsub2(as_h2(lop3_and_or(w, 0x000c000cu, 0x5C005C00u)), as_h2(zm.m[1]));
    d[2] = __hsub2(as_h2(lop3_and_or(w, 0x00300030u, 0x54005400u)), as_h2(zm.m[2]));
    d[3] = __hsub2(as_h2(lop3_and_or(w, 0x00c000c0u, 0x4C004C00u)), as_h2(zm.m[3]));
  }
  template <class F> __device__ static __forceinline__ void unit(const uint4* v, const ZM& zm, F&& f) {
    const uint32_t w[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 d[4];
      half_word(w[j], zm, d);
      f(2 * j, d);
      half_word(w[j] >> 8, zm, d);
      f(2 * j + 1, d);
    }
  }
};

// 3 bits = a 2-bit plane (low bits, laid out exactly like the 2-bit format) plus a 1-bit
// plane whose bits are placed so that a single shift of the plane word lines the high bit
// up with bit (o + 2) of the 2-bit field at offset o: v[0], v[1] are the two 2-bit chunks
// (codes 0..63, 64..127 of the unit) and v[2] the 1-bit chunk (word j covers codes 32j..).
template <> struct Codec<3> {
  using ZM = Codec<2>::ZM;
  __device__ static __forceinline__ ZM zmagic(uint32_t z) { return Codec<2>::zmagic(z); }
  __device__ static __forceinline__ void half_word(uint32_t a, uint32_t b, const ZM& zm, __half2 (&d)[4]) {
    d[0] = __hsub2(as_h2(lop3_or_and(lop3_and_or(a, 0x00030003u, 0x64006400u), b, 0x00040004u)), as_h2(zm.m[0]));
    d[1] = __hsub2(as_h2(lop3_or_and(lop3_and_or(a, 0x000c000cu, 0x5C005C00u), b, 0x00100010u)), as_h2(zm.m[1]));
    d[2] = __hsub2(as_h2(lop3_or_and(lop3_and_or(a, 0x00300030u, 0x54005400u), b, 0x00400040u)), as_h2(zm.m[2]));
    d[3] = __hsub2(as_h2(lop3_or_and(lop3_and_or(a, 0x00c000c0u, 0x4C004C00u), b, 0x01000100u)), as_h2(zm.m[3]));
  }
  template <class F> __device__ static __forceinline__ void unit(const uint4* v, const ZM& zm, F&& f) {
    const uint32_t a[8] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w};
    const uint32_t b[4] = {v[2].x, v[2].y, v[2].z, v[2].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // 32 codes: 2-bit words a[2j], a[2j+1] with plane word b[j]
      __half2 d[4];
      half_word(a[2 * j], b[j] << 2, zm, d);
      f(4 * j, d);
      half_word(a[2 * j] >> 8, b[j] << 1, zm, d);
      f(4 * j + 1, d);
      half_word(a[2 * j + 1], b[j] >> 6, zm, d);
      f(4 * j + 2, d);
      half_word(a[2 * j + 1] >> 8, b[j] >> 7, zm, d);
      f(4 * j + 3, d);
    }
  }
};

// ---------------------------------------------------------------------------
// Fragment layout (4-bit).  One 32-bit word is the A fragment one thread feeds to
// mma.sync.m16n8k16 (weights on the M side): for lane (g = lane / 4, t = lane % 4) of a
// 16-row block it holds rows g and g + 8 at k = 4t .. 4t+3 of a 16-k step:
//   nibble 0: (g, 4t)    nibble 4: (g, 4t+1)    nibble 2: (g, 4t+2)    nibble 6: (g, 4t+3)
//   nibble 1: (g+8, 4t)  nibble 5: (g+8, 4t+1)  nibble 3: (g+8, 4t+2)  nibble 7: (g+8, 4t+3)
// so four ANDs (and one shift) yield the four fragment registers.  A masked nibble is the
// fp16 subnormal q * 2^-24 (bits 0-3 of a half: rows g) or q * 2^-20 (bits 4-7: rows g + 8).
//   qweight  u32 [N/128][2 halves of 64 rows][K/16 steps][32 lanes][4 row blocks]
//   scales   f16 [N/128][K/group][128]   position wt*64 + g*8 + rb*2 + h  <->  row wt*64 + rb*16 + h*8 + g
//   zeros    u8  the same order
// ---------------------------------------------------------------------------
__device__ __forceinline__ void frag4_fields(uint32_t w, uint32_t (&a)[4]) {
  const uint32_t hi = w >> 8;
  a[0] = w & 0x000f000fu;
  a[1] = w & 0x00f000f0u;
  a[2] = hi & 0x000f000fu;
  a[3] = hi & 0x00f000f0u;
}
// The fragment layout for 8 and 2 bits follows the same ownership (lane (g, t) holds rows g and
// g + 8 of each of the four row blocks of a 64-row half, k = 4t .. 4t+3 of a 16-k step):
//   8-bit: two words per row block (row g, row g + 8), byte i = k 4t + i; the row blocks 0,1 of all
//          lanes form one 512-byte chunk of the step, the row blocks 2,3 the next one;
//   2-bit: one word per PAIR of row blocks; the 2-bit field of (row block parity p, row half h,
//          k offset kk) sits at bit 4p + 2h + 16 (kk & 1) + 8 (kk >> 1), so the four fields a row
//          needs share one bit offset inside a half-word (and one power-of-two scale).
//   3-bit: three words per lane and k-step for the four row blocks (96 bits = 32 codes), word j of all lanes
//          a 128-byte plane of the step.  A half-word holds five 3-bit fields (bit offsets 0, 3, 6, 9, 12)
//          and one spare bit.  Row blocks 0..2 live in word rb: rows g at offset 0 (k 4t, 4t+1 in the
//          low / high half-word) and 9 (k 4t+2, 4t+3), rows g + 8 at offsets 3 and 12, so that one
//          shift by 9 brings the second pair of fields onto the first.  Row block 3 takes what is
//          left: offset 6 of word 0 (rows g, k 4t..), word 1 (rows g, k 4t+2..) and word 2 (rows g + 8,
//          k 4t..), and for rows g + 8, k 4t+2.. the spare bits: code bit b is bit 15 (31 for the odd k)
//          of word b.  All its fields are assembled at offset 6.
// FragCodec<BITS>::decode builds the four A-fragment registers of row block rb from the lane's
// words of a k-step; shift_lo / shift_hi are the bit offsets of the fields of rows g / g + 8
// inside a half (the fp16 subnormal they form is q * 2^(shift - 24)).
// word j of a lane and field position of code (rb, h, kk):
// (2-, 4- and 8-bit: a code is one contiguous field; see frag_code_bit for the general form)
__host__ __device__ inline int frag_word_of(int bits, int rb, int h) {
  return bits == 4 ? rb : bits == 8 ? rb * 2 + h : rb >> 1;
}
__host__ __device__ inline int frag_bit_of(int bits, int rb, int h, int kk) {
  if (bits == 8) return 8 * kk;
  if (bits == 4) return 4 * ((kk >> 1) * 2 + (kk & 1) * 4 + h);
  return (rb & 1) * 4 + h * 2 + (kk & 1) * 16 + (kk >> 1) * 8;
}
// word of the lane and bit inside it that hold bit b of code (rb, h, kk), for every bit width
__host__ __device__ inline void frag_code_bit(int bits, int rb, int h, int kk, int b, int* word, int* bit) {
  if (bits != 3) {
    *word = frag_word_of(bits, rb, h);
    *bit = frag_bit_of(bits, rb, h, kk) + b;
    return;
  }
  const int half = (kk & 1) * 16, khi = kk >> 1;
  if (rb < 3) {
    *word = rb;
    *bit = half + h * 3 + khi * 9 + b;
  } else if (h == 1 && khi == 1) {
    *word = b;
    *bit = half + 15;
  } else {
    *word = h == 1 ? 2 : khi;
    *bit = half + 6 + b;
  }
}
template <int BITS> struct FragCodec;
template <> struct FragCodec<3> {
  __device__ static __forceinline__ void decode(const uint32_t* v, int rb, uint32_t (&a)[4]) {
    if (rb < 3) {
      const uint32_t w = v[rb], hi = w >> 9;
      a[0] = w & 0x00070007u;
      a[1] = w & 0x00380038u;
      a[2] = hi & 0x00070007u;
      a[3] = hi & 0x00380038u;
    } else {
      a[0] = v[0] & 0x01C001C0u;
      a[2] = v[1] & 0x01C001C0u;
      a[1] = v[2] & 0x01C001C0u;
      a[3] = ((v[0] >> 9) & 0x00400040u) | ((v[1] >> 8) & 0x00800080u) | ((v[2] >> 7) & 0x01000100u);
    }
  }
  __host__ __device__ static constexpr int shift_lo(int rb) { return rb < 3 ? 0 : 6; }
  __host__ __device__ static constexpr int shift_hi(int rb) { return rb < 3 ? 3 : 6; }
};
template <> struct FragCodec<4> {
  __device__ static __forceinline__ void decode(const uint32_t* v, int rb, uint32_t (&a)[4]) { frag4_fields(v[rb], a); }
  __host__ __device__ static constexpr int shift_lo(int) { return 0; }
  __host__ __device__ static constexpr int shift_hi(int) { return 4; }
};
template <> struct FragCodec<8> {
  __device__ static __forceinline__ void decode(const uint32_t* v, int rb, uint32_t (&a)[4]) {
    a[0] = prmt(v[2 * rb], 0u, 0x4140u);
    a[2] = prmt(v[2 * rb], 0u, 0x4342u);
    a[1] = prmt(v[2 * rb + 1], 0u, 0x4140u);
    a[3] = prmt(v[2 * rb + 1], 0u, 0x4342u);
  }
  __host__ __device__ static constexpr int shift_lo(int) { return 0; }
  __host__ __device__ static constexpr int shift_hi(int) { return 0; }
};
template <> struct FragCodec<2> {
  __device__ static __forceinline__ void decode(const uint32_t* v, int rb, uint32_t (&a)[4]) {
    const uint32_t w = v[rb >> 1], hi = w >> 8;
    const uint32_t m0 = 0x00030003u << ((rb & 1) * 4), m1 = m0 << 2;
    a[0] = w & m0;
    a[1] = w & m1;
    a[2] = hi & m0;
    a[3] = hi & m1;
  }
  __host__ __device__ static constexpr int shift_lo(int rb) { return (rb & 1) * 4; }
  __host__ __device__ static constexpr int shift_hi(int rb) { return (rb & 1) * 4 + 2; }
};
// byte offset of word j of a lane inside the k-step of a 64-row half, and bytes of a k-step
__host__ __device__ inline int frag_word_offset(int bits, int lane, int j) {
  if (bits == 8) return (j >> 2) * 512 + lane * 16 + (j & 3) * 4;
  if (bits == 3) return j * 128 + lane * 4;
  return lane * (4 * bits) + j * 4;
}
__host__ __device__ inline int frag_step_bytes(int bits) { return 128 * bits; }

// row inside the 128-row tile held at position `pos` of the fragment-ordered scale / zero arrays
__host__ __device__ inline int frag_row_of_pos(int pos) {
  return (pos >> 6) * 64 + ((pos >> 1) & 3) * 16 + (pos & 1) * 8 + ((pos >> 3) & 7);
}

// inverse of frag_row_of_pos: where row `r` of a tile sits in the fragment-ordered arrays
__host__ __device__ inline int frag_pos_of_row(int r) {
  return (r >> 6) * 64 + (r & 7) * 8 + ((r >> 4) & 3) * 2 + ((r >> 3) & 1);
}

// Host-visible description of a validated layer (filled by the API layer).
struct LayerView {
  const uint4* qw;
  const __half* qs;     // may be null (group-less)
  const uint8_t* qz;    // may be null (symmetric / group-less)
  int n, k, bits, group_size;
  int npad, tiles, units, groups, units_per_group;
  uint32_t zconst;      // zero used when qz == null
  int layout;           // QFB_LAYOUT_TILE / QFB_LAYOUT_FRAGMENT
};

}  // namespace qfb
