/* Raw-syscall implementation of the liburing subset declared in liburing.h. */
#include "liburing.h"

#include <errno.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

static int sys_setup(unsigned entries, struct io_uring_params *p) {
  return (int)syscall(__NR_io_uring_setup, entries, p);
}

static int sys_enter(int fd, unsigned to_submit, unsigned min_complete, unsigned flags) {
  return (int)syscall(__NR_io_uring_enter, fd, to_submit, min_complete, flags, NULL, 0);
}

int io_uring_queue_init(unsigned entries, struct io_uring *ring, unsigned flags) {
  struct io_uring_params p;
  memset(&p, 0, sizeof(p));
  memset(ring, 0, sizeof(*ring));
  p.flags = flags;
  int fd = sys_setup(entries, &p);
  if (fd < 0) return -errno;

  struct io_uring_sq *sq = &ring->sq;
  struct io_uring_cq *cq = &ring->cq;
  sq->ring_sz = p.sq_off.array + p.sq_entries * sizeof(unsigned);
  cq->ring_sz = p.cq_off.cqes + p.cq_entries * sizeof(struct io_uring_cqe);
  if (p.features & IORING_FEAT_SINGLE_MMAP) {
    if (cq->ring_sz > sq->ring_sz) sq->ring_sz = cq->ring_sz;
    cq->ring_sz = sq->ring_sz;
  }
  sq->ring_ptr = mmap(0, sq->ring_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQ_RING);
  if (sq->ring_ptr == MAP_FAILED) goto fail;
  if (p.features & IORING_FEAT_SINGLE_MMAP) {
    cq->ring_ptr = sq->ring_ptr;
  } else {
    cq->ring_ptr = mmap(0, cq->ring_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_CQ_RING);
    if (cq->ring_ptr == MAP_FAILED) {
      munmap(sq->ring_ptr, sq->ring_sz);
      goto fail;
    }
  }
  sq->sqes = (struct io_uring_sqe *)mmap(0, p.sq_entries * sizeof(struct io_uring_sqe), PROT_READ | PROT_WRITE,
                                         MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQES);
  if (sq->sqes == MAP_FAILED) {
    if (cq->ring_ptr != sq->ring_ptr) munmap(cq->ring_ptr, cq->ring_sz);
    munmap(sq->ring_ptr, sq->ring_sz);
    goto fail;
  }
  char *sp = (char *)sq->ring_ptr, *cp = (char *)cq->ring_ptr;
  sq->khead = (unsigned *)(sp + p.sq_off.head);
  sq->ktail = (unsigned *)(sp + p.sq_off.tail);
  sq->kring_mask = (unsigned *)(sp + p.sq_off.ring_mask);
  sq->kring_entries = (unsigned *)(sp + p.sq_off.ring_entries);
  sq->kflags = (unsigned *)(sp + p.sq_off.flags);
  sq->kdropped = (unsigned *)(sp + p.sq_off.dropped);
  sq->array = (unsigned *)(sp + p.sq_off.array);
  cq->khead = (unsigned *)(cp + p.cq_off.head);
  cq->ktail = (unsigned *)(cp + p.cq_off.tail);
  cq->kring_mask = (unsigned *)(cp + p.cq_off.ring_mask);
  cq->kring_entries = (unsigned *)(cp + p.cq_off.ring_entries);
  cq->koverflow = (unsigned *)(cp + p.cq_off.overflow);
  cq->cqes = (struct io_uring_cqe *)(cp + p.cq_off.cqes);
  /* identity map of the indirection array, as liburing does */
  for (unsigned i = 0; i < p.sq_entries; i++) sq->array[i] = i;
  ring->flags = p.flags;
  ring->features = p.features;
  ring->ring_fd = fd;
  return 0;
fail : {
  int e = errno;
  close(fd);
  errno = e;
  return -e;
}
}

void io_uring_queue_exit(struct io_uring *ring) {
  struct io_uring_sq *sq = &ring->sq;
  struct io_uring_cq *cq = &ring->cq;
  if (sq->sqes) munmap(sq->sqes, *sq->kring_entries * sizeof(struct io_uring_sqe));
  if (cq->ring_ptr && cq->ring_ptr != sq->ring_ptr) munmap(cq->ring_ptr, cq->ring_sz);
  if (sq->ring_ptr) munmap(sq->ring_ptr, sq->ring_sz);
  if (ring->ring_fd >= 0) close(ring->ring_fd);
  ring->ring_fd = -1;
}

struct io_uring_sqe *io_uring_get_sqe(struct io_uring *ring) {
  struct io_uring_sq *sq = &ring->sq;
  unsigned head = __atomic_load_n(sq->khead, __ATOMIC_ACQUIRE);
  if (sq->sqe_tail - head >= *sq->kring_entries) return NULL;
  struct io_uring_sqe *sqe = &sq->sqes[sq->sqe_tail & *sq->kring_mask];
  sq->sqe_tail++;
  return sqe;
}

int io_uring_submit(struct io_uring *ring) {
  struct io_uring_sq *sq = &ring->sq;
  unsigned to_submit = sq->sqe_tail - sq->sqe_head;
  if (to_submit) {
    sq->sqe_head = sq->sqe_tail;
    __atomic_store_n(sq->ktail, sq->sqe_tail, __ATOMIC_RELEASE);
  }
  unsigned pending = *sq->ktail - __atomic_load_n(sq->khead, __ATOMIC_ACQUIRE);
  if (!pending) return 0;
  int rc;
  do {
    rc = sys_enter(ring->ring_fd, pending, 0, 0);
  } while (rc < 0 && errno == EINTR);
  return rc < 0 ? -errno : rc;
}

static unsigned cq_ready(struct io_uring *ring) {
  return __atomic_load_n(ring->cq.ktail, __ATOMIC_ACQUIRE) - *ring->cq.khead;
}

int io_uring_peek_cqe(struct io_uring *ring, struct io_uring_cqe **cqe_ptr) {
  if (!cq_ready(ring)) {
    *cqe_ptr = NULL;
    return -EAGAIN;
  }
  *cqe_ptr = &ring->cq.cqes[*ring->cq.khead & *ring->cq.kring_mask];
  return 0;
}

unsigned io_uring_peek_batch_cqe(struct io_uring *ring, struct io_uring_cqe **cqes, unsigned count) {
  unsigned ready = cq_ready(ring);
  if (ready > count) ready = count;
  unsigned head = *ring->cq.khead, mask = *ring->cq.kring_mask;
  for (unsigned i = 0; i < ready; i++) cqes[i] = &ring->cq.cqes[(head + i) & mask];
  return ready;
}

int io_uring_wait_cqe(struct io_uring *ring, struct io_uring_cqe **cqe_ptr) {
  for (;;) {
    if (io_uring_peek_cqe(ring, cqe_ptr) == 0) return 0;
    int rc = sys_enter(ring->ring_fd, 0, 1, IORING_ENTER_GETEVENTS);
    if (rc < 0 && errno != EINTR) return -errno;
  }
}
