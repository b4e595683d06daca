// Offline packer (replaces qfactory/convert.py:55-81 of the reference) and its inverse.
//
// The packer turns GPTQ-style tensors -- int32 codes [K,N], fp16 scales [K/GS,N], int32
// zeros [K/GS,N] -- into the tile-128 interleaved layout described in qfactory_b200.h.
// The inverse kernels run the SAME Codec<> bit extraction the compute kernels use, so a
// pack -> unpack round trip proves the in-kernel decode bit-exact.
#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

// element held by field f of a 2/4/8-bit word (pair interleave: even elements low half)
__device__ __forceinline__ int field_element(int bits, int f) {
  if (bits == 8) return f;
  const int half_fields = 16 / bits;
  return f < half_fields ? 2 * f : 2 * (f - half_fields) + 1;
}

// bit position of element e (0..31) inside a word of the 3-bit format's 1-bit plane
__device__ __forceinline__ int plane1_bit(int e) {
  const int h = e >> 4, el = e & 15, f = el >> 1, parity = el & 1;
  const int variant = 2 * h + (f >> 2);
  const int base = (variant == 0) ? 0 : (variant == 1) ? 1 : (variant == 2) ? 8 : 9;
  return base + 2 * (f & 3) + 16 * parity;
}

__global__ void pack_weight_kernel(const PackParams p) {
  const int nv = unit_vecs(p.bits);
  const long long total = (long long)p.tiles * p.units * nv * 4 * kTileRows;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int r = (int)(idx % kTileRows);
  long long t = idx / kTileRows;
  const int j = (int)(t % 4); t /= 4;
  const int v = (int)(t % nv); t /= nv;
  const int unit = (int)(t % p.units);
  const int tile = (int)(t / p.units);
  const int n = tile * kTileRows + r;
  const int uk = unit_k(p.bits);
  uint32_t word = 0;
  if (n < p.n) {
    if (p.bits != 3) {
      const int pf = 32 / p.bits;
      const int k0 = unit * uk + j * pf;
      for (int f = 0; f < pf; ++f) {
        const uint32_t q = (uint32_t)p.codes[(size_t)(k0 + field_element(p.bits, f)) * p.n + n];
        word |= (q & ((1u << p.bits) - 1u)) << (f * p.bits);
      }
    } else if (v < 2) {  // 2-bit plane: low two bits of 16 codes
      const int k0 = unit * uk + v * 64 + j * 16;
      for (int f = 0; f < 16; ++f) {
        const uint32_t q = (uint32_t)p.codes[(size_t)(k0 + field_element(2, f)) * p.n + n];
        word |= (q & 3u) << (f * 2);
      }
    } else {  // 1-bit plane: bit 2 of 32 codes
      const int k0 = unit * uk + j * 32;
      for (int e = 0; e < 32; ++e) {
        const uint32_t q = (uint32_t)p.codes[(size_t)(k0 + e) * p.n + n];
        word |= ((q >> 2) & 1u) << plane1_bit(e);
      }
    }
  }
  p.qw[((((size_t)tile * p.units + unit) * nv + v) * kTileRows + r) * 4 + j] = word;
}

__global__ void pack_scale_zero_kernel(const PackParams p) {
  const long long total = (long long)p.tiles * p.groups * kTileRows;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int r = (int)(idx % kTileRows);
  const int g = (int)((idx / kTileRows) % p.groups);
  const int tile = (int)(idx / ((long long)kTileRows * p.groups));
  const int n = tile * kTileRows + r;
  if (p.qs) p.qs[idx] = (n < p.n) ? p.scales[(size_t)g * p.n + n] : __ushort_as_half(0);
  if (p.qz) {
    int z = 0;
    if (n < p.n) {
      z = p.zeros[(size_t)g * p.n + n] + 1;  // GPTQ "zero - 1" convention, clamped like the reference packer
      const int zmax = (1 << p.bits) - 1;
      z = z > zmax ? zmax : z;
    }
    p.qz[idx] = (uint8_t)z;
  }
}

// ---- fragment layouts: one thread per packed word / per scale position --------------------
// word j of lane (g, t) at k-step ks of the 64-row half wt of a tile; frag_word_of / frag_bit_of
// (qfb_common.cuh) say which codes it holds
__global__ void pack_weight_frag_kernel(const PackParams p) {
  const int ksteps = p.k / 16;
  const int wpl = p.bits;  // words per lane and k-step (4 row blocks): 4 * bits bytes
  const long long total = (long long)p.tiles * 2 * ksteps * 32 * wpl;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int j = (int)(idx % wpl);
  long long t = idx / wpl;
  const int lane = (int)(t & 31); t >>= 5;
  const int ks = (int)(t % ksteps); t /= ksteps;
  const int wt = (int)(t & 1);
  const int tile = (int)(t >> 1);
  const int g = lane >> 2, k0 = ks * 16 + 4 * (lane & 3);
  uint32_t word = 0;
  for (int rb = 0; rb < 4; ++rb)
    for (int h = 0; h < 2; ++h) {
      const int n = tile * kTileRows + wt * 64 + rb * 16 + h * 8 + g;
      if (n >= p.n) continue;
      if (p.bits != 3 && frag_word_of(p.bits, rb, h) != j) continue;
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t q = (uint32_t)p.codes[(size_t)(k0 + kk) * p.n + n] & ((1u << p.bits) - 1u);
        if (p.bits != 3) {
          word |= q << frag_bit_of(p.bits, rb, h, kk);
        } else {  // bit by bit: one of the sixteen field pairs of a lane is spread over the spare bits of its three words
          for (int b = 0; b < 3; ++b) {
            int wj, bit;
            frag_code_bit(3, rb, h, kk, b, &wj, &bit);
            if (wj == j) word |= ((q >> b) & 1u) << bit;
          }
        }
      }
    }
  char* base = reinterpret_cast<char*>(p.qw) + ((size_t)(tile * 2 + wt) * ksteps + ks) * frag_step_bytes(p.bits);
  *reinterpret_cast<uint32_t*>(base + frag_word_offset(p.bits, lane, j)) = word;
}

__global__ void pack_scale_zero_frag_kernel(const PackParams p) {
  const long long total = (long long)p.tiles * p.groups * kTileRows;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int pos = (int)(idx % kTileRows);
  const int g = (int)((idx / kTileRows) % p.groups);
  const int tile = (int)(idx / ((long long)kTileRows * p.groups));
  const int n = tile * kTileRows + frag_row_of_pos(pos);
  if (p.qs) p.qs[idx] = (n < p.n) ? p.scales[(size_t)g * p.n + n] : __ushort_as_half(0);
  if (p.qz) {
    int z = 0;
    if (n < p.n) {
      z = p.zeros[(size_t)g * p.n + n] + 1;  // same "zero - 1" convention and clamp as the tile layout
      const int zmax = (1 << p.bits) - 1;
      z = z > zmax ? zmax : z;
    }
    p.qz[idx] = (uint8_t)z;
  }
}

// inverse through FragCodec<BITS>::decode, the extraction the mma kernel itself runs: one thread
// per (lane, k-step, half tile)
template <int BITS>
__global__ void unpack_frag_kernel(const UnpackParams p) {
  using FC = FragCodec<BITS>;
  const int ksteps = p.k / 16;
  const long long total = (long long)p.tiles * 2 * ksteps * 32;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int lane = (int)(idx & 31);
  long long t = idx >> 5;
  const int ks = (int)(t % ksteps); t /= ksteps;
  const int wt = (int)(t & 1);
  const int tile = (int)(t >> 1);
  const int g = lane >> 2;
  const int k0 = ks * 16 + 4 * (lane & 3);
  const char* base = reinterpret_cast<const char*>(p.qw) + ((size_t)(tile * 2 + wt) * ksteps + ks) * frag_step_bytes(BITS);
  uint32_t v[BITS];
#pragma unroll
  for (int j = 0; j < BITS; ++j) v[j] = *reinterpret_cast<const uint32_t*>(base + frag_word_offset(BITS, lane, j));
  const int grp = k0 / (p.k / p.groups);
#pragma unroll
  for (int rb = 0; rb < 4; ++rb) {
    uint32_t a[4];
    FC::decode(v, rb, a);
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // h = 0: row g (registers a[0], a[2]); h = 1: row g + 8 (a[1], a[3])
      const int n = tile * kTileRows + wt * 64 + rb * 16 + h * 8 + g;
      if (n >= p.n) continue;
      const int sh = h ? FC::shift_hi(rb) : FC::shift_lo(rb);
      const uint32_t lo = a[h] >> sh, hi = a[2 + h] >> sh, m = (1u << BITS) - 1u;
      const int q[4] = {(int)(lo & m), (int)((lo >> 16) & m), (int)(hi & m), (int)((hi >> 16) & m)};
      const size_t sz = ((size_t)tile * p.groups + grp) * kTileRows + wt * 64 + g * 8 + rb * 2 + h;
      const __half sc = p.qs ? p.qs[sz] : __ushort_as_half(0x3C00);
      const int z = p.qz ? (int)p.qz[sz] : (int)p.zconst;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (p.codes_out) p.codes_out[(size_t)(k0 + i) * p.n + n] = q[i];
        if (p.w_out) p.w_out[(size_t)(k0 + i) * p.n + n] = __hmul(__int2half_rn(q[i] - z), sc);
      }
    }
  }
}

cudaError_t launch_pack(const PackParams& p, cudaStream_t st) {
  if (p.layout == QFB_LAYOUT_FRAGMENT) {
    const int block = 256;
    const long long total = (long long)p.tiles * 2 * (p.k / 16) * 32 * p.bits;
    pack_weight_frag_kernel<<<(unsigned)((total + block - 1) / block), block, 0, st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (p.qs || p.qz) {
      const long long t2 = (long long)p.tiles * p.groups * kTileRows;
      pack_scale_zero_frag_kernel<<<(unsigned)((t2 + block - 1) / block), block, 0, st>>>(p);
      e = cudaGetLastError();
    }
    return e;
  }
  const int nv = unit_vecs(p.bits);
  const long long total = (long long)p.tiles * p.units * nv * 4 * kTileRows;
  const int block = 256;
  pack_weight_kernel<<<(unsigned)((total + block - 1) / block), block, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (p.qs || p.qz) {
    const long long t2 = (long long)p.tiles * p.groups * kTileRows;
    pack_scale_zero_kernel<<<(unsigned)((t2 + block - 1) / block), block, 0, st>>>(p);
    e = cudaGetLastError();
  }
  return e;
}

template <int BITS>
__global__ void unpack_kernel(const UnpackParams p) {
  using G = Geo<BITS>;
  using C = Codec<BITS>;
  const long long total = (long long)p.tiles * p.units * kTileRows;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int r = (int)(idx % kTileRows);
  const int unit = (int)((idx / kTileRows) % p.units);
  const int tile = (int)(idx / ((long long)kTileRows * p.units));
  const int n = tile * kTileRows + r;
  if (n >= p.n) return;
  uint4 v[G::kUnitVecs];
#pragma unroll
  for (int i = 0; i < G::kUnitVecs; ++i)
    v[i] = ldg_stream_v4(p.qw + (((size_t)tile * p.units + unit) * G::kUnitVecs + i) * kTileRows + r);
  const int k0 = unit * G::kUnitK;
  if (p.codes_out) {
    const typename C::ZM zm = C::zmagic(0);
    C::unit(v, zm, [&](int j8, __half2(&d)[4]) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(d[i]);
        p.codes_out[(size_t)(k0 + j8 * 8 + 2 * i) * p.n + n] = (int32_t)f.x;
        p.codes_out[(size_t)(k0 + j8 * 8 + 2 * i + 1) * p.n + n] = (int32_t)f.y;
      }
    });
  }
  if (p.w_out) {
    const int g = unit / p.units_per_group;
    const size_t sz = ((size_t)tile * p.groups + g) * kTileRows + r;
    const __half2 s2 = __half2half2(p.qs ? p.qs[sz] : __ushort_as_half(0x3C00));
    const typename C::ZM zm = C::zmagic(p.qz ? (uint32_t)p.qz[sz] : p.zconst);
    C::unit(v, zm, [&](int j8, __half2(&d)[4]) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 w = __hmul2(d[i], s2);
        p.w_out[(size_t)(k0 + j8 * 8 + 2 * i) * p.n + n] = __low2half(w);
        p.w_out[(size_t)(k0 + j8 * 8 + 2 * i + 1) * p.n + n] = __high2half(w);
      }
    });
  }
}

// fp16 weight [K, N] -> group-wise asymmetric codes, scales and GPTQ-convention zeros, the front end
// of "construct a layer from an fp16 weight" (reference: tests/acc_gptq.py:10-29).  One thread per
// (group, column); every operation is rounded to fp16 exactly where the reference's fp16 tensor
// expression rounds (each division and product computed in fp32 and rounded once), so the result
// equals the framework expression bit for bit.
__device__ __forceinline__ __half h_div(__half a, __half b) { return __float2half_rn(__half2float(a) / __half2float(b)); }
__device__ __forceinline__ __half h_mul(__half a, float b) { return __float2half_rn(__half2float(a) * b); }

__global__ void quantize_kernel(const __half* __restrict__ w, int k, int n, int group_size, int levels,
                                int32_t* __restrict__ codes, __half* __restrict__ scales, int32_t* __restrict__ zeros) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int groups = k / group_size;
  if (idx >= (long long)groups * n) return;
  const int col = (int)(idx % n), g = (int)(idx / n);
  const __half* src = w + (size_t)g * group_size * n + col;
  __half wmax = src[0], wmin = src[0];
  for (int i = 1; i < group_size; ++i) {
    const __half v = src[(size_t)i * n];
    wmax = __hmax(wmax, v);
    wmin = __hmin(wmin, v);
  }
  const __half span = __hsub_rn(wmax, wmin);
  scales[idx] = __float2half_rn(__half2float(span) / (float)levels);
  // zero = trunc(max(-min / span * levels - 1, 0))
  const __half zf = __hsub_rn(h_mul(h_div(__hneg(wmin), span), (float)levels), __float2half_rn(1.f));
  zeros[idx] = (int32_t)__half2float(__hmax(zf, __float2half_rn(0.f)));
  for (int i = 0; i < group_size; ++i) {
    const __half q = h_mul(h_div(__hsub_rn(src[(size_t)i * n], wmin), span), (float)levels);
    codes[(size_t)(g * group_size + i) * n + col] = (int32_t)__half2float(q);
  }
}

cudaError_t launch_quantize(const __half* w, int k, int n, int bits, int group_size, int32_t* codes, __half* scales,
                            int32_t* zeros, cudaStream_t st) {
  const long long total = (long long)(k / group_size) * n;
  quantize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(w, k, n, group_size, (1 << bits) - 1, codes, scales,
                                                                    zeros);
  return cudaGetLastError();
}

cudaError_t launch_unpack(const UnpackParams& p, cudaStream_t st) {
  if (p.layout == QFB_LAYOUT_FRAGMENT) {
    const int block = 256;
    const long long tf = (long long)p.tiles * 2 * (p.k / 16) * 32;
    const unsigned gridf = (unsigned)((tf + block - 1) / block);
    if (p.bits == 4) unpack_frag_kernel<4><<<gridf, block, 0, st>>>(p);
    else if (p.bits == 8) unpack_frag_kernel<8><<<gridf, block, 0, st>>>(p);
    else if (p.bits == 2) unpack_frag_kernel<2><<<gridf, block, 0, st>>>(p);
    else if (p.bits == 3) unpack_frag_kernel<3><<<gridf, block, 0, st>>>(p);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
  }
  const long long total = (long long)p.tiles * p.units * kTileRows;
  const int block = 128;
  const unsigned grid = (unsigned)((total + block - 1) / block);
  switch (p.bits) {
    case 2: unpack_kernel<2><<<grid, block, 0, st>>>(p); break;
    case 3: unpack_kernel<3><<<grid, block, 0, st>>>(p); break;
    case 4: unpack_kernel<4><<<grid, block, 0, st>>>(p); break;
    case 8: unpack_kernel<8><<<grid, block, 0, st>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace qfb
