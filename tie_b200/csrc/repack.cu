// Upload-time re-ordering of Q6_K tensors into the "R8" layout.
//
// A Q6_K super-block is 210 bytes (gguf.h:101-106), so rows of packed blocks are only 2-byte
// aligned and cannot be read with 128-bit loads.  Groups of 8 consecutive rows are 16-byte
// aligned, so within each group the bytes are re-ordered (same byte count, nothing added):
//   [quant chunks: (row, block, part) x 48 B][scales: (row, block, part) x 4 B][d: (row, block) x 2 B]
// where part = (half n, slice l16) and a chunk holds the three 16-byte pieces one lane needs for
// 64 weights: ql[64n+16*l16..], ql[64n+32+16*l16..], qh[32n+16*l16..]; the 4 scales of a part are
// scales[8n + l16 + {0,2,4,6}].  Element order and values are unchanged.
#include "common.cuh"
#include "kernels.cuh"

namespace tie {

__global__ void __launch_bounds__(256) repack_q6k_r8(const uint8_t *__restrict__ raw, uint8_t *__restrict__ dst,
						     size_t n_units, int nb)
{
	// unit = (row, block, part)
	size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (u >= n_units)
		return;
	const int part = (int)(u & 3);
	const size_t rb = u >> 2;
	const int b = (int)(rb % nb);
	const size_t row = rb / nb;
	const int n = part >> 1, l16 = part & 1;
	const uint8_t *blk = raw + (row * nb + b) * Q6K_BYTES;
	uint8_t *grp = dst + (row >> 3) * q6k_r8_group_bytes(nb);
	const int r8 = (int)(row & 7);
	uint8_t *ch = grp + q6k_r8_chunk_off(nb, r8, b, part);
	const uint8_t *ql = blk, *qh = blk + 128, *sc = blk + 192;
	for (int i = 0; i < 16; i++) {
		ch[i] = ql[64 * n + 16 * l16 + i];
		ch[16 + i] = ql[64 * n + 32 + 16 * l16 + i];
		ch[32 + i] = qh[32 * n + 16 * l16 + i];
	}
	uint8_t *so = grp + q6k_r8_scale_off(nb, r8, b, part);
	for (int j = 0; j < 4; j++)
		so[j] = sc[8 * n + l16 + 2 * j];
	if (part == 0) {
		uint8_t *dd = grp + q6k_r8_d_off(nb, r8, b);
		dd[0] = blk[208];
		dd[1] = blk[209];
	}
}

int launch_repack_q6k_r8(tie_cuda_ctx *c, const uint8_t *raw, uint8_t *dst, size_t n_rows_total, int nb)
{
	size_t units = n_rows_total * nb * 4;
	repack_q6k_r8<<<(unsigned)((units + 255) / 256), 256, 0, c->stream>>>(raw, dst, units, nb);
	TIE_CUDA_LAUNCHED(c);
	return TIE_CUDA_OK;
}

}  // namespace tie
