/*
 * sage_b200 — C ABI of the all-reduce that follows a row-parallel packed linear when a model
 * is sharded over the GPUs of one node (o_proj and down_proj under tensor parallelism).
 *
 * The reference's packed inference is single-GPU (benchmarks/model.py loads one model on one
 * device), so nothing here replaces a reference function; the row/column tags the sharding
 * follows are those of weight_vq/blockwise/artifacts.py:10-18.
 *
 * One process per GPU.  Every rank owns an EXCHANGE: one device allocation that its peers map
 * through CUDA IPC.  An all-reduce is one kernel per rank, no library collective:
 *
 *   push    each CTA stores its chunk of this rank's partial rows into slot [parity][rank] of
 *           EVERY peer's exchange (plain stores over NVLink), then publishes the call's epoch in
 *           the peer's flag [rank][cta] with a system-scope release;
 *   wait    it polls the flags the peers publish in its OWN exchange (local memory) until all
 *           carry the epoch - a bounded wait: after two seconds the kernel records
 *           SAGEB200_ERR_TIMEOUT in the device's status word and returns;
 *   reduce  it sums the W partials in rank order in FP32 (its own from registers, the others
 *           from its own exchange), rounds once to FP16 and writes the result in place.
 *
 * Every rank adds the same numbers in the same order, so all ranks hold identical results.
 * Epochs and the slot parity live in device memory and advance by one per call, so the call
 * can be captured in a CUDA graph and replayed; every rank must make the same sequence of calls
 * (same element counts).  A slot is written again two calls later, which a peer can only reach
 * after this rank has published the call in between, i.e. after its reads of the slot are over.
 *
 * Every function returns SAGEB200_OK (0) or a negative SAGEB200_ERR_* code of sage_b200.h.
 */
#ifndef SAGE_B200_PEER_H_
#define SAGE_B200_PEER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAGEB200_PEER_MAX_WORLD 8
#define SAGEB200_PEER_HANDLE_BYTES 64

/* Bytes of an exchange that all-reduces up to `capacity` FP16 elements (a multiple of 8) among
 * `world` ranks; 0 for arguments out of range. */
size_t sageb200_peer_exchange_bytes(int world, long long capacity);

/* Allocates and zeroes this rank's exchange on the current device (cudaMalloc: a set-up call,
 * outside any stream capture) and writes the 64-byte IPC handle the peers open. */
int sageb200_peer_create(int world, long long capacity, void **exchange, unsigned char *handle);

/* Maps a peer's exchange into this process (enables peer access on first use). */
int sageb200_peer_open(const unsigned char *handle, void **exchange);

/* Unmaps a peer's exchange / frees this rank's own.  The caller makes sure (a host barrier) that
 * no rank still runs a kernel that touches it. */
int sageb200_peer_close(void *peer_exchange);
int sageb200_peer_destroy(void *own_exchange);

/*
 * data[elements] (FP16, device memory of this rank, 16-byte aligned, elements a multiple of 8
 * and at most `capacity`) becomes the sum over the ranks of their `data`, in place.
 * `exchanges[r]` is rank r's exchange as mapped in this process (`exchanges[rank]` the own one).
 * One launch on `stream`.
 */
int sageb200_peer_all_reduce(void *const *exchanges, int world, int rank, long long capacity, void *data,
                             long long elements, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_PEER_H_ */
