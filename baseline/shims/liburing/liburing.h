/* Minimal stand-in for liburing, for building the reference KV manager on an image that has the
 * kernel's io_uring UAPI header but not the liburing package. It covers exactly the calls that the
 * reference's SSD layer makes (queue init/exit, get_sqe, prep read/write/readv/writev, submit,
 * peek/wait/advance of completions) on top of the raw io_uring_setup / io_uring_enter syscalls.
 * Single-issuer use only, as in the reference (one ring per IO thread). */
#pragma once
#include <linux/io_uring.h>
#include <stdint.h>
#include <string.h>
#include <sys/uio.h>

#ifdef __cplusplus
extern "C" {
#endif

struct io_uring_sq {
  unsigned *khead, *ktail, *kring_mask, *kring_entries, *kflags, *kdropped, *array;
  struct io_uring_sqe *sqes;
  unsigned sqe_head, sqe_tail;
  size_t ring_sz;
  void *ring_ptr;
};

struct io_uring_cq {
  unsigned *khead, *ktail, *kring_mask, *kring_entries, *koverflow;
  struct io_uring_cqe *cqes;
  size_t ring_sz;
  void *ring_ptr;
};

struct io_uring {
  struct io_uring_sq sq;
  struct io_uring_cq cq;
  unsigned flags;
  int ring_fd;
  unsigned features;
};

int io_uring_queue_init(unsigned entries, struct io_uring *ring, unsigned flags);
void io_uring_queue_exit(struct io_uring *ring);
struct io_uring_sqe *io_uring_get_sqe(struct io_uring *ring);
int io_uring_submit(struct io_uring *ring);
int io_uring_wait_cqe(struct io_uring *ring, struct io_uring_cqe **cqe_ptr);
int io_uring_peek_cqe(struct io_uring *ring, struct io_uring_cqe **cqe_ptr);
unsigned io_uring_peek_batch_cqe(struct io_uring *ring, struct io_uring_cqe **cqes, unsigned count);

static inline void io_uring_cq_advance(struct io_uring *ring, unsigned nr) {
  if (nr) __atomic_store_n(ring->cq.khead, *ring->cq.khead + nr, __ATOMIC_RELEASE);
}

static inline void io_uring_cqe_seen(struct io_uring *ring, struct io_uring_cqe *cqe) {
  if (cqe) io_uring_cq_advance(ring, 1);
}

static inline void io_uring_prep_rw(int op, struct io_uring_sqe *sqe, int fd, const void *addr,
                                    unsigned len, uint64_t offset) {
  memset(sqe, 0, sizeof(*sqe));
  sqe->opcode = (uint8_t)op;
  sqe->fd = fd;
  sqe->off = offset;
  sqe->addr = (uint64_t)(uintptr_t)addr;
  sqe->len = len;
}

static inline void io_uring_prep_read(struct io_uring_sqe *sqe, int fd, void *buf, unsigned nbytes,
                                      uint64_t offset) {
  io_uring_prep_rw(IORING_OP_READ, sqe, fd, buf, nbytes, offset);
}

static inline void io_uring_prep_write(struct io_uring_sqe *sqe, int fd, const void *buf, unsigned nbytes,
                                       uint64_t offset) {
  io_uring_prep_rw(IORING_OP_WRITE, sqe, fd, buf, nbytes, offset);
}

static inline void io_uring_prep_readv(struct io_uring_sqe *sqe, int fd, const struct iovec *iovecs,
                                       unsigned nr_vecs, uint64_t offset) {
  io_uring_prep_rw(IORING_OP_READV, sqe, fd, iovecs, nr_vecs, offset);
}

static inline void io_uring_prep_writev(struct io_uring_sqe *sqe, int fd, const struct iovec *iovecs,
                                        unsigned nr_vecs, uint64_t offset) {
  io_uring_prep_rw(IORING_OP_WRITEV, sqe, fd, iovecs, nr_vecs, offset);
}

#ifdef __cplusplus
}
#endif
