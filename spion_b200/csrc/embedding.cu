// Weight gradient of a token embedding with a small table (models/model_transformer.py: nn.Embedding(vocab_size,
// embedding_dim), vocab_size 256 - 512 in the benchmark tasks):  dW[v, :] = sum over tokens t with ids[t] == v of g[t, :].
//
// The framework sorts the token ids (radix sort + segmented reduction, several launches) because its table may have
// any size.  Here the whole table fits in shared memory: a CTA (one per SM) walks a contiguous chunk of tokens in order,
// staged through shared memory in batches, and adds each gradient row to the table row of its id; the partial tables of
// the CTAs are then summed in CTA order.  Every addition has a fixed place in a fixed sequence, so the result is the
// same bits on every run.  HBM-bound: the gradient rows are read once.
#include "common.cuh"

namespace {

constexpr int EMB_THREADS = 1024;                  // 32 warps
constexpr int EMB_BATCH_BYTES = 32 * 1024;          // gradient rows of one staged batch (32 - 128 tokens)
constexpr int EMB_STAGES = 3;                      // batches in flight or in use
constexpr int EMB_MAX_TABLE_FLOATS = 24 * 1024;    // 96 KB of shared memory for the table

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(PENDING)); }

// Shared memory: table [V][N] fp32, then EMB_STAGES stages of { gradient rows [batch][N], ids [batch] }.
// The batch of a stage arrives by 16-byte asynchronous copies issued by all threads, EMB_STAGES - 1 batches ahead.
// Warp w owns the 32 columns (w % (N/32)) * 32 ... of the table rows whose id % groups == w / (N/32), groups =
// 32 / (N/32): a table element is only ever touched by one thread, in token order.  A warp reads the 32 ids of a
// sub-batch at once, votes on the ones that are its own and walks those; a run of equal ids is summed in a register
// before it goes to the table (padding tokens come in long runs).
__host__ __device__ inline int emb_batch(int N, int esize) {   // tokens per staged batch: a multiple of 32
  const int b = EMB_BATCH_BYTES / (N * esize);
  return b > 128 ? 128 : (b < 32 ? 32 : b / 32 * 32);
}

template <typename TG>
__global__ void __launch_bounds__(EMB_THREADS) embedding_bwd_kernel(const long long* __restrict__ ids,
                                                                    const TG* __restrict__ g, long long T, int V,
                                                                    int N, float* __restrict__ partial) {
  const int batch = emb_batch(N, (int)sizeof(TG));
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* table = reinterpret_cast<float*>(smem_raw);
  const size_t stage_bytes = (size_t)batch * N * sizeof(TG) + batch * sizeof(long long);
  unsigned char* stages = smem_raw + (size_t)V * N * sizeof(float);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col_parts = N / 32, groups = (EMB_THREADS / 32) / col_parts;
  const int col = (warp % col_parts) * 32 + lane, grp = warp / col_parts;

  for (int i = threadIdx.x; i < V * N; i += EMB_THREADS) table[i] = 0.f;

  // this CTA's tokens: whole batches, so that every copy starts on a 16-byte boundary
  const long long batches = (T + batch - 1) / batch;
  const long long per = (batches + gridDim.x - 1) / gridDim.x;
  const long long b0 = (long long)blockIdx.x * per, b1 = min(batches, b0 + per);

  auto fetch = [&](long long b) {
    unsigned char* st = stages + (size_t)((b - b0) % EMB_STAGES) * stage_bytes;
    const long long t0 = b * batch;
    const int ntok = (int)min((long long)batch, T - t0);
    const int row_pieces = N * (int)sizeof(TG) / 16;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(g + t0 * N);
    for (int i = threadIdx.x; i < ntok * row_pieces; i += EMB_THREADS) cp_async16(st + (size_t)i * 16, src + (size_t)i * 16);
    unsigned char* sid = st + (size_t)batch * N * sizeof(TG);
    const unsigned char* isrc = reinterpret_cast<const unsigned char*>(ids + t0);
    for (int i = threadIdx.x; i < ntok / 2; i += EMB_THREADS) cp_async16(sid + (size_t)i * 16, isrc + (size_t)i * 16);
    if ((ntok & 1) && threadIdx.x == 0)   // odd tail: the last id by a plain load
      reinterpret_cast<long long*>(sid)[ntok - 1] = ids[t0 + ntok - 1];
  };

  int cur = -1;
  float acc = 0.f;
  for (int k = 0; k < EMB_STAGES - 1; ++k) {
    if (b0 + k < b1) fetch(b0 + k);
    cp_async_commit();
  }
  for (long long b = b0; b < b1; ++b) {
    if (b + EMB_STAGES - 1 < b1) fetch(b + EMB_STAGES - 1);
    cp_async_commit();
    cp_async_wait<EMB_STAGES - 1>();
    __syncthreads();                      // batch b has landed for every thread (and the table is zeroed)
    const unsigned char* st = stages + (size_t)((b - b0) % EMB_STAGES) * stage_bytes;
    const TG* gs = reinterpret_cast<const TG*>(st);
    const long long* sid = reinterpret_cast<const long long*>(st + (size_t)batch * N * sizeof(TG));
    const int ntok = (int)min((long long)batch, T - b * batch);
    for (int s = 0; s < ntok; s += 32) {
      long long raw = -1;
      if (s + lane < ntok) raw = sid[s + lane];
      const bool mine = raw >= 0 && raw < V && ((int)raw & (groups - 1)) == grp;   // groups is a power of two
      unsigned m = __ballot_sync(0xffffffffu, mine);
      auto add = [&](int id, float v) {
        if (id == cur) {
          acc += v;
        } else {
          if (cur >= 0) table[cur * N + col] += acc;
          cur = id;
          acc = v;
        }
      };
      while (m) {                          // two tokens per turn: their loads do not wait for each other
        const int k0 = __ffs(m) - 1;
        m &= m - 1;
        const int k1 = m ? __ffs(m) - 1 : k0;
        const bool two = m != 0;
        m &= m - 1;
        const int id0 = __shfl_sync(0xffffffffu, (int)raw, k0), id1 = __shfl_sync(0xffffffffu, (int)raw, k1);
        const float v0 = to_f32(gs[(s + k0) * N + col]), v1 = to_f32(gs[(s + k1) * N + col]);
        add(id0, v0);
        if (two) add(id1, v1);
      }
    }
    __syncthreads();                      // the stage may be overwritten by the next fetch
  }
  if (cur >= 0) table[cur * N + col] += acc;
  __syncthreads();
  float* out = partial + (long long)blockIdx.x * V * N;
  for (int i = threadIdx.x; i < V * N; i += EMB_THREADS) out[i] = table[i];
}

// dW[i] = sum of the partial tables in a fixed order: warp w of a CTA adds parts w, w + 8, ... for 32 consecutive
// table entries, the eight sums meet in shared memory and are added in warp order.
__global__ void __launch_bounds__(256) embedding_bwd_reduce_kernel(const float* __restrict__ partial, int parts,
                                                                   int table_floats, float* __restrict__ dW) {
  __shared__ float s_part[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (i < table_floats)
    for (int p = warp; p < parts; p += 8) s += partial[(long long)p * table_floats + i];
  s_part[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && i < table_floats) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += s_part[w][lane];
    dW[i] = t;
  }
}

// out[t, :] = tok[ids[t], :] + pos[t % L, :]: token and position embedding of the encoder input in one pass (the
// framework gathers, then adds the broadcast position rows in a second kernel).  One thread per four columns; both
// tables stay in cache, so the kernel is bound by writing out.  ids outside [0, V) give the position row alone.
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const long long* __restrict__ ids, const float* __restrict__ tok,
                                                            const float* __restrict__ pos, float* __restrict__ out,
                                                            long long T, int L, int V, int N) {
  const int per_row = N >> 2;
  const long long total = T * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 4;
    const long long id = ids[t];
    float4 v = *reinterpret_cast<const float4*>(pos + (size_t)(t % L) * N + c);
    if (id >= 0 && id < V) {
      const float4 w = *reinterpret_cast<const float4*>(tok + (size_t)id * N + c);
      v.x += w.x, v.y += w.y, v.z += w.z, v.w += w.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)t * N + c) = v;
  }
}

size_t emb_smem(int V, int N, int g_is_bf16) {
  const int batch = emb_batch(N, g_is_bf16 ? 2 : 4);
  return (size_t)V * N * sizeof(float) + EMB_STAGES * ((size_t)batch * N * (g_is_bf16 ? 2 : 4) + batch * sizeof(long long));
}

int emb_grid(long long T) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  const long long want = (T + 255) / 256;   // at least 256 tokens per CTA
  return (int)std::max<long long>(1, std::min<long long>(sms, want));
}

}  // namespace

// Floats of workspace spion_embedding_backward needs for T tokens: one partial table per CTA.
extern "C" long long spion_embedding_workspace_floats(long long T, int V, int N) {
  if (T < 1 || V < 1 || N < 1) return 0;
  const int grid = emb_grid(T);
  return grid < 1 ? 0 : (long long)grid * V * N;
}

// dW [V, N] fp32 = scatter-sum of the gradient rows g [T, N] (fp32 or bf16, 16-byte aligned) by token id (int64,
// 16-byte aligned; ids outside [0, V) are skipped).  N in {32, 64, 128, 256}, V * N <= 24576 (table plus three
// staged batches of at most 32 KB of rows within the shared memory of an SM).  Overwrites dW.
// Fixed summation order.
extern "C" int spion_embedding_backward(const long long* ids, const void* g, int g_is_bf16, long long T, int V, int N,
                                        float* dW, float* workspace, void* cuda_stream) {
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  if (!ids || !g || !dW || !workspace || T < 1) return SPION_ERR_ARG;
  if ((((uintptr_t)ids) | ((uintptr_t)g)) & 15) return SPION_ERR_ARG;
  if ((N != 32 && N != 64 && N != 128 && N != 256) || V < 1 || (long long)V * N > EMB_MAX_TABLE_FLOATS)
    return SPION_ERR_SHAPE;
  const int grid = emb_grid(T);
  if (grid < 1) return SPION_ERR_CUDA;
  const size_t smem = emb_smem(V, N, g_is_bf16);
  if (smem > 227 * 1024) return SPION_ERR_SHAPE;
  if (g_is_bf16) {
    SPION_CUDA_TRY(cudaFuncSetAttribute(embedding_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    embedding_bwd_kernel<__nv_bfloat16><<<grid, EMB_THREADS, smem, stream>>>(ids, (const __nv_bfloat16*)g, T, V, N,
                                                                             workspace);
  } else {
    SPION_CUDA_TRY(cudaFuncSetAttribute(embedding_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    embedding_bwd_kernel<float><<<grid, EMB_THREADS, smem, stream>>>(ids, (const float*)g, T, V, N, workspace);
  }
  SPION_LAUNCH_CHECK();
  embedding_bwd_reduce_kernel<<<(V * N + 31) / 32, 256, 0, stream>>>(workspace, grid, V * N, dW);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}

// out [T, N] fp32 = tok[ids[t]] + pos[t % L] (tok [V, N], pos [>= L, N], all 16-byte aligned, N a multiple of 4):
// the input of the first encoder layer before dropout (models/model_transformer.py: token embedding plus position
// embedding of positions 0 .. L-1 for every sequence of the batch; T = batch * L).
extern "C" int spion_embedding_forward(const long long* ids, const float* tok, const float* pos, float* out, long long T,
                                       int L, int V, int N, void* cuda_stream) {
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  if (!ids || !tok || !pos || !out || T < 1 || L < 1 || V < 1) return SPION_ERR_ARG;
  if ((((uintptr_t)tok) | ((uintptr_t)pos) | ((uintptr_t)out)) & 15) return SPION_ERR_ARG;
  if (N < 4 || N % 4 != 0) return SPION_ERR_SHAPE;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return SPION_ERR_CUDA;
  const long long want = (T * (N / 4) + 255) / 256;
  const int grid = (int)std::max<long long>(1, std::min<long long>(want, (long long)sms * 8));
  embedding_fwd_kernel<<<grid, 256, 0, stream>>>(ids, tok, pos, out, T, L, V, N);
  SPION_LAUNCH_CHECK();
  return SPION_OK;
}
