// Test infrastructure: a declaration-only stand-in for liburing, so that the reference's headers (which include it from
// common/file_io.hpp) can be PARSED on a machine without the library.  Nothing here is ever called.
#pragma once
#include <cstdint>
struct io_uring {
	int ring_fd;
};
struct io_uring_sqe {
	uint64_t user_data;
};
struct io_uring_cqe {
	uint64_t user_data;
	int32_t res;
};
int io_uring_queue_init(unsigned entries, io_uring* ring, unsigned flags);
void io_uring_queue_exit(io_uring* ring);
io_uring_sqe* io_uring_get_sqe(io_uring* ring);
void io_uring_prep_read(io_uring_sqe* sqe, int fd, void* buf, unsigned nbytes, uint64_t offset);
void io_uring_prep_write(io_uring_sqe* sqe, int fd, const void* buf, unsigned nbytes, uint64_t offset);
void io_uring_sqe_set_data(io_uring_sqe* sqe, void* data);
void* io_uring_cqe_get_data(const io_uring_cqe* cqe);
int io_uring_submit(io_uring* ring);
int io_uring_wait_cqe(io_uring* ring, io_uring_cqe** cqe_ptr);
void io_uring_cqe_seen(io_uring* ring, io_uring_cqe* cqe);
