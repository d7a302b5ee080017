// seqgemm_tc.cuh -- the layer-list products on the 5th-generation tensor cores (bf16 mode, many tokens):
//   D[128 weight rows][128 tokens] += W_tile . X_tile^T with tcgen05.mma (kind::f16 on bf16 operands, cta_group::1),
//   fp32 accumulators in TMEM.  Both operands are K-major bf16 matrices in global memory (weights as stored,
//   activations as the producing kernels wrote them) and come in by TMA (cp.async.bulk.tensor, SWIZZLE_128B; edges of M,
//   N and K are zero-filled by the copy).  One lane issues the copies, one lane the MMAs, completion flows through
//   mbarriers (tcgen05.commit); four warps read the accumulators back (tcgen05.ld) and apply the epilogue of the product:
//   fp32 store, activation-type store, or Dynamic-Tanh + residual add.  blockIdx.z walks a batch of per-head products
//   (3-D tensor maps; an operand shared by the batch keeps a 2-D map).
// Every wait is bounded: a stalled pipeline records a code in `err`, every role falls through to the common exit, TMEM
// is released and the host reports the code after the step.
#pragma once

#include <map>
#include <tuple>

#include "seqkernels.cuh"
#include "tc05.cuh"

#define TG_BM 128
#define TG_BN 128
#define TG_BK 64
#define TG_STAGES 3
#define TG_THREADS 192
#define TG_STAGE_BYTES ((TG_BM + TG_BN) * TG_BK * 2)
#define TG_SMEM (TG_STAGES * TG_STAGE_BYTES + 1024)
// kind::f16 instruction descriptor: D = f32 (bit 4), A = B = bf16 (bits 7, 10), both K-major, N at bit 17 (>> 3), M at bit 24 (>> 4)
#define TG_IDESC ((1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TG_BN >> 3) << 17) | ((uint32_t)(TG_BM >> 4) << 24))

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
	asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)), "l"(map),
	             "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
	             : "memory");
}
// about a second at most; false = gave up
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
	for (unsigned spins = 0; spins < (1u << 24); ++spins)
		if (mbar_try_wait(bar, parity)) return true;
	return false;
}

__global__ void __launch_bounds__(TG_THREADS) k_seq_gemm_tc(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmArgs a, int w3d, int x3d,
                                                             int* err) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	extern __shared__ unsigned char smem_dyn[];
	__shared__ __align__(8) uint64_t full[TG_STAGES], empty[TG_STAGES], accum;
	__shared__ uint32_t tmem_base_s;
	unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int m0 = blockIdx.x * TG_BM, n0 = blockIdx.y * TG_BN, z = blockIdx.z;
	const int nkb = (a.K + TG_BK - 1) / TG_BK;
	const GemmRows gr = gemm_rows(a, z);
	if (n0 >= gr.count) return; // a grouped product's tile past the end of its group (uniform over the CTA, before any barrier or TMEM allocation)
	auto a_tile = [&](int s) { return smem + (size_t)s * TG_STAGE_BYTES; };
	auto b_tile = [&](int s) { return smem + (size_t)s * TG_STAGE_BYTES + TG_BM * TG_BK * 2; };
	if (tid == 0) {
		for (int s = 0; s < TG_STAGES; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], 1);
		mbar_init(&accum, 1);
		mbar_init_fence();
	}
	if (warp == 1) tmem_alloc(&tmem_base_s, TG_BN);
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_base_s;

	if (warp == 0) {
		if (lane == 0) {
			for (int kb = 0; kb < nkb; ++kb) {
				const int s = kb % TG_STAGES;
				if (!mbar_wait_bounded(&empty[s], ((kb / TG_STAGES) & 1) ^ 1)) {
					atomicExch(err, 1);
					break;
				}
				mbar_expect_tx(&full[s], TG_STAGE_BYTES);
				if (w3d) tma_load_3d(a_tile(s), &tm_w, kb * TG_BK, m0, z, &full[s]);
				else tma_load_2d(a_tile(s), &tm_w, kb * TG_BK, m0, &full[s]);
				if (x3d) tma_load_3d(b_tile(s), &tm_x, kb * TG_BK, n0, z, &full[s]);
				else tma_load_2d(b_tile(s), &tm_x, kb * TG_BK, gr.base + n0, &full[s]); // rows past the group are other groups' (or zero fill): never stored
			}
		}
	} else if (warp == 1) {
		if (lane == 0) {
			bool ok = true;
			for (int kb = 0; kb < nkb && ok; ++kb) {
				const int s = kb % TG_STAGES;
				if (!mbar_wait_bounded(&full[s], (kb / TG_STAGES) & 1)) {
					atomicExch(err, 2);
					ok = false;
					break;
				}
				tc_fence_after();
#pragma unroll
				for (int k = 0; k < TG_BK / 16; ++k) // 16 bf16 = 32 bytes along K inside the swizzle atom: +2 in the 16-byte address field
					umma_f16(tmem_base, umma_desc_sw128(a_tile(s)) + 2 * k, umma_desc_sw128(b_tile(s)) + 2 * k, TG_IDESC, (kb | k) ? 1u : 0u);
				umma_commit(&empty[s]);
			}
			umma_commit(&accum); // arrives when everything issued so far has completed, also after a stall
		}
	} else {
		const bool ok = mbar_wait_bounded(&accum, 0);
		if (!ok && lane == 0) atomicExch(err, 3);
		tc_fence_after();
		if (ok) {
			const int q4 = warp & 3; // the TMEM lane quarter this warp may read
			const int m = m0 + q4 * 32 + lane;
			for (int c0 = 0; c0 < TG_BN; c0 += 32) {
				if (n0 + c0 >= gr.count) break;
				float v[32];
				tmem_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + c0, v);
#pragma unroll
				for (int j = 0; j < 32; ++j) gemm_store<bf16>(a, z, gr, n0 + c0 + j, m, v[j]); // lanes = consecutive weight rows: coalesced
			}
		}
		tc_fence_before();
	}
	__syncthreads();
	if (warp == 1) {
		tc_fence_after();
		tmem_dealloc(tmem_base, TG_BN);
	}
}

// ---------------------------------------------------------------- host side
typedef CUresult (*TgEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct TgState {
	TgEncodeFn encode = nullptr;
	int* err_host = nullptr; // pinned + mapped
	int* err_dev = nullptr;
	std::map<std::tuple<const void*, long, long, long, long, int>, CUtensorMap> maps;
};
static TgState g_tg;

static inline void gemm_tc_setup() {
	if (g_tg.encode) return;
	cudaDriverEntryPointQueryResult qres;
	void* fn = nullptr;
	CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
	if (!fn || qres != cudaDriverEntryPointSuccess) CALM_FATAL("cuTensorMapEncodeTiled is not available from this driver");
	g_tg.encode = (TgEncodeFn)fn;
	CUDA_CHECK(cudaHostAlloc((void**)&g_tg.err_host, sizeof(int), cudaHostAllocMapped));
	*g_tg.err_host = 0;
	CUDA_CHECK(cudaHostGetDevicePointer((void**)&g_tg.err_dev, g_tg.err_host, 0));
	CUDA_CHECK(cudaFuncSetAttribute(k_seq_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, TG_SMEM));
}
// a stalled pipeline leaves its code here; read after the stream has been synchronised
static inline int gemm_tc_error() { return g_tg.err_host ? *g_tg.err_host : 0; }

// bf16 [batch][rows][cols] with row stride ld and batch stride bs (elements); box = 64 columns x `box_rows` rows
static inline const CUtensorMap* tg_map(const void* base, long rows, long cols, long ld, long bs, int batch, int box_rows) {
	const auto key = std::make_tuple(base, rows, cols, ld, bs, batch * 1024 + box_rows);
	auto it = g_tg.maps.find(key);
	if (it != g_tg.maps.end()) return &it->second;
	if (g_tg.maps.size() > 8192) g_tg.maps.clear();
	CUtensorMap m;
	const bool three = bs != 0 && batch > 1;
	const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
	const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)bs * 2};
	const cuuint32_t box[3] = {TG_BK, (cuuint32_t)box_rows, 1}, estr[3] = {1, 1, 1};
	CUresult r = g_tg.encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, three ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
	                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS) return nullptr; // a layout the copy engine does not describe: the caller keeps the mma.sync kernel
	return &(g_tg.maps[key] = m);
}

// shapes the kernel takes: enough tokens to fill its tiles (a matrix of few rows, a router's, fills the rest of its tile with the copy's zeros), 16-byte aligned rows and bases
static inline bool gemm_tc_fits(const GemmArgs& a, int batch) {
	auto al8 = [](long v) { return v % 8 == 0; };
	return a.N >= 64 && a.M >= 8 && a.K >= 32 && al8(a.ldx) && al8(a.ldw) && al8(a.xbs) && al8(a.wbs) && ((uintptr_t)a.X & 15) == 0 && ((uintptr_t)a.W & 15) == 0 &&
	       batch < 65536;
}
// false: no tensor map for one of the operands, nothing was launched
static inline bool gemm_tc_launch(const GemmArgs& a, int batch, cudaStream_t stream) {
	const CUtensorMap* mw = tg_map(a.W, a.M, a.K, a.ldw, a.wbs, batch, TG_BM);
	const CUtensorMap* mx = tg_map(a.X, a.seg ? a.x_rows : a.N, a.K, a.ldx, a.xbs, batch, TG_BN);
	if (!mw || !mx) return false;
	const dim3 grid((a.M + TG_BM - 1) / TG_BM, (a.N + TG_BN - 1) / TG_BN, batch);
	k_seq_gemm_tc<<<grid, TG_THREADS, TG_SMEM, stream>>>(*mw, *mx, a, a.wbs != 0 && batch > 1, a.xbs != 0 && batch > 1, g_tg.err_dev);
	return true;
}
