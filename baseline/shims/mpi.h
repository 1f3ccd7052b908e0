// Single-process stand-in for <mpi.h>, just large enough to build the reference's unmodified sources for
// one rank (its single-node engines, loaders and CPU executor).  Rank 0 of a world of size 1: collectives are
// no-ops, point-to-point calls have no peer and abort.  Not an MPI implementation; used only by the baseline
// build under baseline/, never by the framework itself.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cstring>

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef long MPI_Aint;
typedef int MPI_Request;
typedef int MPI_Op;
struct MPI_Status { int MPI_SOURCE; int MPI_TAG; int MPI_ERROR; };

#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_THREAD_SINGLE 0
#define MPI_THREAD_FUNNELED 1
#define MPI_THREAD_SERIALIZED 2
#define MPI_THREAD_MULTIPLE 3
#define MPI_ANY_SOURCE (-1)
#define MPI_ANY_TAG (-1)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)
#define MPI_MAX_PROCESSOR_NAME 256
#define MPI_IN_PLACE ((void*)1)

#define MPI_CHAR 1
#define MPI_UNSIGNED_CHAR 2
#define MPI_INT 3
#define MPI_UNSIGNED 4
#define MPI_LONG 5
#define MPI_UNSIGNED_LONG 6
#define MPI_FLOAT 7
#define MPI_DOUBLE 8
#define MPI_INT8_T 9
#define MPI_INT32_T 10
#define MPI_UINT16_T 11
#define MPI_UINT32_T 12
#define MPI_UINT64_T 13
#define MPI_SUM 1
#define MPI_MAX 2
#define MPI_MIN 3

static inline int mpi_single_no_peer(const char* what) {
    std::fprintf(stderr, "mpi_single: %s needs a second rank; this build runs one process only\n", what);
    std::abort();
    return 1;
}
static inline int mpi_single_sizeof(MPI_Datatype t) {
    switch (t) {
        case MPI_CHAR: case MPI_UNSIGNED_CHAR: case MPI_INT8_T: return 1;
        case MPI_UINT16_T: return 2;
        case MPI_INT: case MPI_UNSIGNED: case MPI_FLOAT: case MPI_INT32_T: case MPI_UINT32_T: return 4;
        default: return 8;
    }
}

static inline int MPI_Init(int*, char***) { return MPI_SUCCESS; }
static inline int MPI_Init_thread(int*, char***, int required, int* provided) { if (provided) *provided = required; return MPI_SUCCESS; }
static inline int MPI_Finalize() { return MPI_SUCCESS; }
static inline int MPI_Comm_rank(MPI_Comm, int* r) { *r = 0; return MPI_SUCCESS; }
static inline int MPI_Comm_size(MPI_Comm, int* s) { *s = 1; return MPI_SUCCESS; }
static inline int MPI_Get_processor_name(char* name, int* len) { std::strcpy(name, "localhost"); *len = 9; return MPI_SUCCESS; }
static inline int MPI_Barrier(MPI_Comm) { return MPI_SUCCESS; }
static inline int MPI_Bcast(void*, int, MPI_Datatype, int, MPI_Comm) { return MPI_SUCCESS; }
static inline int MPI_Allreduce(const void* in, void* out, int n, MPI_Datatype t, MPI_Op, MPI_Comm) {
    if (in != MPI_IN_PLACE && in != out) std::memcpy(out, in, (size_t)n * mpi_single_sizeof(t));
    return MPI_SUCCESS;
}
static inline int MPI_Allgather(const void* in, int n, MPI_Datatype t, void* out, int, MPI_Datatype, MPI_Comm) {
    if (in != MPI_IN_PLACE && in != out) std::memcpy(out, in, (size_t)n * mpi_single_sizeof(t));
    return MPI_SUCCESS;
}
static inline int MPI_Send(const void*, int, MPI_Datatype, int, int, MPI_Comm) { return mpi_single_no_peer("MPI_Send"); }
static inline int MPI_Recv(void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Status*) { return mpi_single_no_peer("MPI_Recv"); }
static inline int MPI_Isend(const void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request*) { return mpi_single_no_peer("MPI_Isend"); }
static inline int MPI_Irecv(void*, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request*) { return mpi_single_no_peer("MPI_Irecv"); }
static inline int MPI_Test(MPI_Request*, int* flag, MPI_Status*) { *flag = 0; return MPI_SUCCESS; }
static inline int MPI_Wait(MPI_Request*, MPI_Status*) { return mpi_single_no_peer("MPI_Wait"); }
static inline int MPI_Cancel(MPI_Request*) { return MPI_SUCCESS; }
static inline int MPI_Request_free(MPI_Request*) { return MPI_SUCCESS; }
static inline int MPI_Get_count(const MPI_Status*, MPI_Datatype, int* c) { *c = 0; return MPI_SUCCESS; }
static inline int MPI_Get_address(const void* p, MPI_Aint* a) { *a = (MPI_Aint)p; return MPI_SUCCESS; }
static inline int MPI_Type_create_struct(int, const int*, const MPI_Aint*, const MPI_Datatype*, MPI_Datatype* t) { *t = 100; return MPI_SUCCESS; }
static inline int MPI_Type_commit(MPI_Datatype*) { return MPI_SUCCESS; }
static inline int MPI_Abort(MPI_Comm, int code) { std::exit(code); return MPI_SUCCESS; }
