// KV compressor tiles: softmax-gated pooling of per-token records into
// compressed entries, decomposed for context parallelism.  Every rank reduces
// the window slots it owns to per-channel statistics (m, l, w), bulk-pushes
// them from shared memory to the entry's owner rank and bumps the sequence's
// event cell on every rank; the owner merges the statistics, applies RMS norm,
// rope on the last 64 channels, and quantises into its pools.
//
// Tiles for the 256 worker threads of a block (a stand-alone kernel of 256 threads, or warps 0..7 of a
// persistent block), one sequence per call.  Channel c of the 512-wide stream
// is handled by thread c % 256 (two channels per thread), the 128-wide indexer
// stream by threads 0..127.  All exponentials are expf (not the fast
// approximation): the pooled values are compared with an fp32 CPU oracle.
#pragma once

#include "comm.cuh"
#include "events.cuh"

namespace mdc {

constexpr int kHdAttn = 512, kHdIdx = 128, kRope = 64, kRingDefault = 8;
// slots of the record ring: the caller's ring_slots (>= ceil(8 / cp): the window holds 8 tokens, cp-interleaved), 8 when 0
__device__ __host__ inline int ring_slots_of(const mdc_compress_params& p) { return p.ring_slots > 0 ? p.ring_slots : kRingDefault; }
constexpr int kRecAttn = 4 * kHdAttn, kRecIdx = 4 * kHdIdx, kRecOnline = 2 * kHdAttn;
// statistics payload, in floats: [valid, entry, -, -][m|l|w attn][m|l|w idx]
constexpr int kSMa = 4, kSLa = kSMa + kHdAttn, kSWa = kSLa + kHdAttn;
constexpr int kSMi = kSWa + kHdAttn, kSLi = kSMi + kHdIdx, kSWi = kSLi + kHdIdx;
constexpr int kCsaStatsF = kSWi + kHdIdx;        // 1924 floats = 7696 bytes
constexpr int kOnlStatsF = 4 + 3 * kHdAttn;      // 1540 floats = 6160 bytes
constexpr float kNegBig = -1.0e30f;
constexpr float kHadamardScale = 0.0883883461356163f;  // fp32 nearest of 1/sqrt(128)

__device__ inline PeerBuffer as_peer(const mdc_peer_buffer& a) {
  return PeerBuffer{static_cast<unsigned char*>(a.base), a.offsets, a.my_rank, a.world, a.mc_base};
}
__device__ inline EventSet as_events(const mdc_event_set& e) {
  return EventSet{static_cast<unsigned char*>(e.base), e.offsets, e.my_rank, e.world};
}
__device__ inline int stats_floats(int ratio) { return ratio == 4 ? kCsaStatsF : kOnlStatsF; }

// position this rank owns in the step [s, s + q_len), or -1
__device__ inline int my_position(int s, int q_len, int cp, int rank) {
  const int p = s + ((rank - s) % cp + cp) % cp;
  return p < s + q_len ? p : -1;
}
// first position in [s, s + q_len) that closes a group of `ratio` tokens, or -1
__device__ inline int closing_position(int s, int q_len, int ratio) {
  for (int p = s; p < s + q_len; ++p)
    if ((p + 1) % ratio == 0) return p;
  return -1;
}

// OWN_EVENTS: the tile posts the notifies itself (stand-alone kernels).  Inside the persistent kernel the
// task's notify edges do that, after the push has completed here.
template <bool OWN_EVENTS>
__device__ inline void push_stats_and_notify(const mdc_compress_params& p, int b, int owner, bool closed, float* stage,
                                             int n_floats) {
  const PeerBuffer arena = as_peer(p.arena);
  const EventSet ev = as_events(p.events);
  fence_proxy_async_smem();
  sync_workers();
  if (threadIdx.x == 0) {
    if (closed && p.do_push) {
      const int64_t off = p.stats_off + (static_cast<int64_t>(b) * p.cp + p.rank) * n_floats * 4;
      push_start(arena.peer_ptr(off, owner), stage, n_floats * 4);
      push_finish();
    }
    if (OWN_EVENTS) {
      __threadfence_system();
      for (int dst = 0; dst < p.cp; ++dst) ev.notify_1t(p.ev_base_id + b, dst);
    }
  }
}

// ---------------------------------------------------------------- window machine (ratio 4)
// stage: kCsaStatsF floats of shared memory, 16-byte aligned
template <bool OWN_EVENTS>
__device__ inline void csa_step_tile(const mdc_compress_params& p, int b, float* stage) {
  const int tid = threadIdx.x;
  const int kRing = ring_slots_of(p);
  const int s = p.seq_len[b];
  const int mine = my_position(s, p.q_len, p.cp, p.rank);
  if (mine >= 0) {  // append this rank's new record to its ring
    const int slot = (mine / p.cp) % kRing;
    for (int i = tid; i < kRecAttn; i += kBlockThreads)
      p.ring_attn[(static_cast<int64_t>(b) * kRing + slot) * kRecAttn + i] = p.new_attn[static_cast<int64_t>(b) * kRecAttn + i];
    for (int i = tid; i < kRecIdx; i += kBlockThreads)
      p.ring_idx[(static_cast<int64_t>(b) * kRing + slot) * kRecIdx + i] = p.new_idx[static_cast<int64_t>(b) * kRecIdx + i];
  }
  sync_workers();
  const int pc = closing_position(s, p.q_len, 4);
  const bool closed = pc >= 0;
  const int n = closed ? pc >> 2 : 0;
  if (closed) {
    // statistics over the window slots this rank owns: slot j <-> token 4n-4+j, role j / 4
    for (int stream = 0; stream < 2; ++stream) {
      const int hd = stream ? kHdIdx : kHdAttn;
      const float* ring = stream ? p.ring_idx : p.ring_attn;
      const float* ape = stream ? p.ape_idx : p.ape_attn;
      const int rec = 4 * hd;
      for (int ch = tid; ch < hd; ch += kBlockThreads) {
        float m = kNegBig;
        float sc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int tok = 4 * n - 4 + j;
          sc[j] = kNegBig;
          if (tok >= 0 && tok % p.cp == p.rank) {
            const float* r = ring + (static_cast<int64_t>(b) * kRing + (tok / p.cp) % kRing) * rec;
            sc[j] = r[(2 + (j >> 2)) * hd + ch] + ape[j * hd + ch];
            m = fmaxf(m, sc[j]);
          }
        }
        float l = 0.f, w = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int tok = 4 * n - 4 + j;
          if (tok >= 0 && tok % p.cp == p.rank) {
            const float* r = ring + (static_cast<int64_t>(b) * kRing + (tok / p.cp) % kRing) * rec;
            const float e = expf(sc[j] - m);
            l += e;
            w += e * r[(j >> 2) * hd + ch];
          }
        }
        const int base = stream ? kSMi : kSMa;
        stage[base + ch] = m;
        stage[base + hd + ch] = l;
        stage[base + 2 * hd + ch] = w;
      }
    }
  }
  if (tid == 0) {
    stage[0] = closed ? 1.f : 0.f;
    stage[1] = static_cast<float>(n);
    stage[2] = stage[3] = 0.f;
  }
  push_stats_and_notify<OWN_EVENTS>(p, b, n % p.cp, closed, stage, kCsaStatsF);
}

// ---------------------------------------------------------------- online machine (ratio 64 / 128)
__device__ inline void online_fold(const mdc_compress_params& p, int b, int pos, int ch) {
  float* st = p.state + static_cast<int64_t>(b) * 3 * kHdAttn;
  const float kv = p.new_attn[static_cast<int64_t>(b) * kRecOnline + ch];
  const float sc = p.new_attn[static_cast<int64_t>(b) * kRecOnline + kHdAttn + ch] + p.ape_attn[(pos % p.ratio) * kHdAttn + ch];
  const float m_old = st[ch], l_old = st[kHdAttn + ch], k_old = st[2 * kHdAttn + ch];
  const float m_new = fmaxf(m_old, sc);
  const float keep = l_old * expf(m_old - m_new);
  const float add = expf(sc - m_new);
  const float l_new = keep + add;
  st[ch] = m_new;
  st[kHdAttn + ch] = l_new;
  st[2 * kHdAttn + ch] = (k_old * keep + kv * add) / l_new;
}

// stage: kOnlStatsF floats of shared memory, 16-byte aligned
template <bool OWN_EVENTS>
__device__ inline void online_step_tile(const mdc_compress_params& p, int b, float* stage) {
  const int tid = threadIdx.x;
  const int s = p.seq_len[b];
  const int mine = my_position(s, p.q_len, p.cp, p.rank);
  const int pc = closing_position(s, p.q_len, p.ratio);
  const bool closed = pc >= 0;
  const int n = closed ? pc / p.ratio : 0;
  float* st = p.state + static_cast<int64_t>(b) * 3 * kHdAttn;
  for (int ch = tid; ch < kHdAttn; ch += kBlockThreads) {
    if (mine >= 0 && (!closed || mine <= pc)) online_fold(p, b, mine, ch);   // token of the closing chunk
    if (closed) {
      stage[4 + ch] = st[ch];
      stage[4 + kHdAttn + ch] = st[kHdAttn + ch];
      stage[4 + 2 * kHdAttn + ch] = st[2 * kHdAttn + ch];
      st[ch] = kNegBig;
      st[kHdAttn + ch] = 0.f;
      st[2 * kHdAttn + ch] = 0.f;
    }
    if (mine >= 0 && closed && mine > pc) online_fold(p, b, mine, ch);       // token of the next chunk
  }
  if (tid == 0) {
    stage[0] = closed ? 1.f : 0.f;
    stage[1] = static_cast<float>(n);
    stage[2] = stage[3] = 0.f;
  }
  push_stats_and_notify<OWN_EVENTS>(p, b, n % p.cp, closed, stage, kOnlStatsF);
}

// ---------------------------------------------------------------- finalize helpers
// Block-wide sum in double precision.  The squares of fp32 values are exact in fp64 and their
// fp64 sum is accurate far below one fp32 ulp, so the fp32 result does not depend on the order of
// the reduction: a CPU restatement that accumulates in fp64 gets the same bits.
__device__ inline double block_sum_f64(double v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  sync_workers();
  if (lane == 0) red[warp] = v;
  sync_workers();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += red[w];
  return t;
}

__device__ inline uint32_t e2m1_code(float q) {
  const float a = fabsf(q);
  uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
  return c | (q < 0.f ? 8u : 0u);
}

// merged statistic of channel `ch` over the cp payloads of sequence b (system-scope loads)
__device__ inline float merge_channel(const float* stats, int cp, int n_floats, int m_off, int l_off, int w_off, int ch,
                                      bool online) {
  float m = kNegBig;
  for (int r = 0; r < cp; ++r) m = fmaxf(m, ld_sys_f32(stats + r * n_floats + m_off + ch));
  float num = 0.f, den = 0.f;
  for (int r = 0; r < cp; ++r) {
    const float* s = stats + r * n_floats;
    const float f = expf(ld_sys_f32(s + m_off + ch) - m);
    const float l = ld_sys_f32(s + l_off + ch) * f;
    const float w = ld_sys_f32(s + w_off + ch);
    den += l;
    num += online ? w * l : w * f;   // online state carries the normalised kv, the window machine the raw sum
  }
  return num / den;
}

// RMS norm + rope(last 64 channels at position pos) of an hd-wide vector held
// one or two channels per thread; result in y_smem[hd]
__device__ inline void norm_rope(float v0, float v1, int hd, const float* norm_w, float eps, const float* freqs, int pos,
                                 float* y_smem, double* red) {
  // Every step rounds exactly like the fp32 tensor arithmetic of the reference chain
  // (compress_ref.py:77-95): mean of squares (accumulated in fp64, see block_sum_f64), + eps,
  // 1 / sqrt with IEEE division and square root, x * factor * weight as two multiplications,
  // and the rotation as two rounded products and one rounded sum (no fused multiply-add).
  const int tid = threadIdx.x;
  const bool two = hd > kBlockThreads;
  double ssq = 0.0;
  if (tid < hd) ssq = static_cast<double>(v0) * v0 + (two ? static_cast<double>(v1) * v1 : 0.0);
  const float mean = static_cast<float>(block_sum_f64(ssq, red) / static_cast<double>(hd));
  const float factor = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  if (tid < hd) {
    y_smem[tid] = __fmul_rn(__fmul_rn(v0, factor), norm_w[tid]);
    if (two) y_smem[tid + kBlockThreads] = __fmul_rn(__fmul_rn(v1, factor), norm_w[tid + kBlockThreads]);
  }
  sync_workers();
  float r[2];
  for (int k = 0; k < (two ? 2 : 1); ++k) {
    const int ch = tid + k * kBlockThreads;
    r[k] = 0.f;
    if (ch < hd && ch >= hd - kRope) {
      const int i2 = ch - (hd - kRope);
      const float c = freqs[static_cast<int64_t>(pos) * kRope + (i2 & ~1)];
      const float sn = freqs[static_cast<int64_t>(pos) * kRope + (i2 | 1)];
      // even channel: re * c - im * s ; odd channel: re * s + im * c
      r[k] = __fadd_rn(__fmul_rn(y_smem[ch], c), __fmul_rn(y_smem[ch ^ 1], (ch & 1) ? sn : -sn));
    }
  }
  sync_workers();
  for (int k = 0; k < (two ? 2 : 1); ++k) {
    const int ch = tid + k * kBlockThreads;
    if (ch < hd && ch >= hd - kRope) y_smem[ch] = r[k];
  }
  sync_workers();
}

__device__ inline void store_attn_entry(const mdc_compress_params& p, int b, int slot, const float* y) {
  const int tid = threadIdx.x;  // two consecutive channels per thread
  const int ch = 2 * tid;
  const int64_t off = (static_cast<int64_t>(b) * p.max_entries + slot) * kHdAttn + ch;
  if (p.attn_pool_dtype == MDC_DT_E4M3) {
    const float a = fminf(fmaxf(y[ch] * p.inv_fp8_scale, -448.f), 448.f);
    const float c = fminf(fmaxf(y[ch + 1] * p.inv_fp8_scale, -448.f), 448.f);
    uint16_t pk;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(c), "f"(a));
    *reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(p.attn_pool) + off) = pk;
  } else {
    __nv_bfloat162 t = __floats2bfloat162_rn(y[ch], y[ch + 1]);
    *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(p.attn_pool) + off) = t;
  }
}

__device__ inline void fp4_quant_warp(const float (&x)[4], uint8_t* data, uint8_t* sf, int fmt);

// warp 0: staged 128-point Hadamard of y[0..127] (4 consecutive elements per
// lane: strides 1, 2 in-thread, then lane masks 1..16), scaled, then block-scaled FP4 (fp4_quant_warp).
__device__ inline void hadamard_quant_warp(const float* y, uint8_t* data, uint8_t* sf, int fmt) {
  const int lane = threadIdx.x & 31;
  const float x0 = y[4 * lane], x1 = y[4 * lane + 1], x2 = y[4 * lane + 2], x3 = y[4 * lane + 3];
  const float b0 = x0 + x1, b1 = x0 - x1, b2 = x2 + x3, b3 = x2 - x3;
  float d[4] = {b0 + b2, b1 + b3, b0 - b2, b1 - b3};
#pragma unroll
  for (int msk = 1; msk < 32; msk <<= 1) {
    const bool hi = (lane & msk) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, d[i], msk);
      d[i] = hi ? o - d[i] : d[i] + o;
    }
  }
  float q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = d[i] * kHadamardScale;
  fp4_quant_warp(q, data, sf, fmt);
}

// One warp quantises a 128-wide vector (lane l holds elements 4l .. 4l+3) to block-scaled FP4: values
// rounded through bf16, scale from the block maximum / 6 (MXFP4: UE8M0 ceil per 32 elements; NVFP4:
// UE4M3 round-to-nearest per 16), E2M1 codes with ties to the even code.  Writes 64 code bytes at `data`
// and the scales at `sf` (MXFP4: one byte per 8 lanes at sf[lane/8]; NVFP4: per 4 lanes at sf[lane/4]).
__device__ inline void fp4_quant_warp(const float (&x)[4], uint8_t* data, uint8_t* sf, int fmt) {
  const int lane = threadIdx.x & 31;
  float q[4], amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    q[i] = __bfloat162float(__float2bfloat16_rn(x[i]));
    amax = fmaxf(amax, fabsf(q[i]));
  }
  const int group_lanes = (fmt == MDC_FMT_MXFP4) ? 8 : 4;
  for (int msk = 1; msk < group_lanes; msk <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, msk));
  float scale;
  uint8_t sf_byte;
  if (fmt == MDC_FMT_MXFP4) {
    const float sc = fmaxf(amax / 6.f, 1e-4f);
    const uint32_t bits = __float_as_uint(sc);
    const int e = static_cast<int>((bits >> 23) & 255) - 127 + ((bits & 0x7fffffu) != 0 ? 1 : 0);
    scale = __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
    sf_byte = static_cast<uint8_t>(min(max(e + 127, 0), 254));
  } else {
    uint16_t pk;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.f), "f"(fminf(amax / 6.f, 448.f)));
    sf_byte = static_cast<uint8_t>(pk & 0xff);
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(pk));
    scale = __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xffff)));
  }
  uint32_t nib[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) nib[i] = (scale > 0.f) ? e2m1_code(q[i] / fmaxf(scale, 1.953125e-3f)) : 0u;
  data[2 * lane] = static_cast<uint8_t>(nib[0] | (nib[1] << 4));
  data[2 * lane + 1] = static_cast<uint8_t>(nib[2] | (nib[3] << 4));
  if ((lane % group_lanes) == 0) sf[lane / group_lanes] = sf_byte;
}

// owner-side wait for the cp statistics of sequence b; false = gave up
__device__ inline bool wait_stats(const mdc_compress_params& p, int b, int* flag) {
  if (threadIdx.x == 0) {
    const EventSet ev = as_events(p.events);
    unsigned long long seen = 0;
    const unsigned long long want = static_cast<unsigned long long>(p.cp) * (static_cast<unsigned long long>(p.phase) + 1ull);
    *flag = 1;
    if (!ev.poll_1t(p.ev_base_id + b, want, p.cp > 1, p.wait_budget_ns, &seen)) {
      report_failure(p.status, MDC_DEV_WAIT_TIMEOUT, p.ev_base_id + b, b, seen, want);
      *flag = 0;
    }
  }
  sync_workers();
  return *flag != 0;
}

}  // namespace mdc

namespace mdc {

struct FinalizeSmem {
  double red[kWarps];
  float y[kHdAttn];
  int flag;
};

// ratio 4, owner of entry n: merge both streams, post chains, pool writes.  OWN_EVENTS: the tile
// waits for the cp statistics itself; inside the persistent kernel the task's wait edge has done so.
template <bool OWN_EVENTS>
__device__ inline void csa_finalize_tile(const mdc_compress_params& p, int b, FinalizeSmem& sm) {
  const int tid = threadIdx.x;
  const int s = p.seq_len[b];
  const int pc = closing_position(s, p.q_len, 4);
  if (pc < 0) return;
  const int n = pc >> 2;
  if (n % p.cp != p.rank) return;
  if (OWN_EVENTS && !wait_stats(p, b, &sm.flag)) return;
  const int slot = n / p.cp;
  if (slot >= p.max_entries || 4 * n >= p.freq_rows) {
    if (tid == 0) report_failure(p.status, MDC_DEV_BAD_INDEX, slot, n, 0, 0);
    return;
  }
  const float* stats = reinterpret_cast<const float*>(static_cast<const unsigned char*>(p.arena.base) + p.stats_off) +
                       static_cast<int64_t>(b) * p.cp * kCsaStatsF;
  // attention stream: channels tid and tid + 256
  const float a0 = merge_channel(stats, p.cp, kCsaStatsF, kSMa, kSLa, kSWa, tid, false);
  const float a1 = merge_channel(stats, p.cp, kCsaStatsF, kSMa, kSLa, kSWa, tid + kBlockThreads, false);
  if (p.dbg_attn) {
    float* d = p.dbg_attn + (static_cast<int64_t>(b) * p.max_entries + slot) * kHdAttn;
    d[tid] = a0;
    d[tid + kBlockThreads] = a1;
  }
  norm_rope(a0, a1, kHdAttn, p.norm_w_attn, p.norm_eps, p.freqs, 4 * n, sm.y, sm.red);
  store_attn_entry(p, b, slot, sm.y);
  sync_workers();
  // indexer stream: channel tid < 128
  float i0 = 0.f;
  if (tid < kHdIdx) {
    i0 = merge_channel(stats, p.cp, kCsaStatsF, kSMi, kSLi, kSWi, tid, false);
    if (p.dbg_idx) p.dbg_idx[(static_cast<int64_t>(b) * p.max_entries + slot) * kHdIdx + tid] = i0;
  }
  norm_rope(i0, 0.f, kHdIdx, p.norm_w_idx, p.norm_eps, p.freqs, 4 * n, sm.y, sm.red);
  if (tid < 32 && p.idx_pool) {
    const int P = p.idx_page_tokens;
    const int sf_per_tok = (p.idx_fmt == MDC_FMT_MXFP4) ? 4 : 8;
    const int page_bytes = P * 64 + P * sf_per_tok;
    uint8_t* pg = p.idx_pool + (static_cast<int64_t>(b) * (p.max_entries / P) + slot / P) * page_bytes;
    const int tok = slot % P;
    uint8_t* sf = (p.idx_fmt == MDC_FMT_MXFP4) ? pg + P * 64 + (tok % 32) * 16 + (tok / 32) * 4 : pg + P * 64 + tok * 8;
    hadamard_quant_warp(sm.y, pg + tok * 64, sf, p.idx_fmt);
  }
  if (tid == 0 && p.k_valid) p.k_valid[b] = slot + 1;
}

// online machine, owner of entry n: merge the cp states, post chain, pool write
template <bool OWN_EVENTS>
__device__ inline void online_finalize_tile(const mdc_compress_params& p, int b, FinalizeSmem& sm) {
  const int tid = threadIdx.x;
  const int s = p.seq_len[b];
  const int pc = closing_position(s, p.q_len, p.ratio);
  if (pc < 0) return;
  const int n = pc / p.ratio;
  if (n % p.cp != p.rank) return;
  if (OWN_EVENTS && !wait_stats(p, b, &sm.flag)) return;
  const int slot = n / p.cp;
  if (slot >= p.max_entries || n * p.ratio >= p.freq_rows) {
    if (tid == 0) report_failure(p.status, MDC_DEV_BAD_INDEX, slot, n, 0, 0);
    return;
  }
  const float* stats = reinterpret_cast<const float*>(static_cast<const unsigned char*>(p.arena.base) + p.stats_off) +
                       static_cast<int64_t>(b) * p.cp * kOnlStatsF;
  const float a0 = merge_channel(stats, p.cp, kOnlStatsF, 4, 4 + kHdAttn, 4 + 2 * kHdAttn, tid, true);
  const float a1 = merge_channel(stats, p.cp, kOnlStatsF, 4, 4 + kHdAttn, 4 + 2 * kHdAttn, tid + kBlockThreads, true);
  if (p.dbg_attn) {
    float* d = p.dbg_attn + (static_cast<int64_t>(b) * p.max_entries + slot) * kHdAttn;
    d[tid] = a0;
    d[tid + kBlockThreads] = a1;
  }
  norm_rope(a0, a1, kHdAttn, p.norm_w_attn, p.norm_eps, p.freqs, n * p.ratio, sm.y, sm.red);
  store_attn_entry(p, b, slot, sm.y);
  if (tid == 0 && p.k_valid) p.k_valid[b] = slot + 1;
}

}  // namespace mdc
