// Stand-in for <mpi.h>: the subset of MPI that the reference uses, for ranks that are processes of one machine.
// Implemented in mpi_shim.cc over Unix-domain sockets (abstract namespace); rank, size and job name come from the
// environment that baseline/shims/mpirun_local.py sets (MPISHIM_RANK, MPISHIM_SIZE, MPISHIM_JOB).  Without that
// environment a process is rank 0 of a world of size 1.  Messages are eager (a receiver thread drains every socket
// into a mailbox), matching is by (source, tag) in arrival order, and every call may be made from several threads
// (the reference asks for MPI_THREAD_MULTIPLE).  Only MPI_COMM_WORLD exists.  Not an MPI implementation: used by the
// baseline build under baseline/ only, never by the framework itself.
#pragma once
#include <stddef.h>

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef long MPI_Aint;
typedef int MPI_Request;
typedef int MPI_Op;
struct MPI_Status { int MPI_SOURCE; int MPI_TAG; int MPI_ERROR; long count_bytes_; };

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
#define MPI_REQUEST_NULL (-1)

#define MPI_DATATYPE_NULL 0
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
#define MPI_BYTE 14
#define MPI_INT64_T 15
#define MPI_SUM 1
#define MPI_MAX 2
#define MPI_MIN 3

int MPI_Init(int* argc, char*** argv);
int MPI_Init_thread(int* argc, char*** argv, int required, int* provided);
int MPI_Finalize();
int MPI_Abort(MPI_Comm comm, int code);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Get_processor_name(char* name, int* len);
int MPI_Barrier(MPI_Comm comm);
int MPI_Bcast(void* buf, int count, MPI_Datatype type, int root, MPI_Comm comm);
int MPI_Allreduce(const void* in, void* out, int count, MPI_Datatype type, MPI_Op op, MPI_Comm comm);
int MPI_Allgather(const void* in, int count, MPI_Datatype type, void* out, int rcount, MPI_Datatype rtype, MPI_Comm comm);
int MPI_Send(const void* buf, int count, MPI_Datatype type, int dest, int tag, MPI_Comm comm);
int MPI_Recv(void* buf, int count, MPI_Datatype type, int source, int tag, MPI_Comm comm, MPI_Status* status);
int MPI_Isend(const void* buf, int count, MPI_Datatype type, int dest, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Irecv(void* buf, int count, MPI_Datatype type, int source, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Test(MPI_Request* req, int* flag, MPI_Status* status);
int MPI_Wait(MPI_Request* req, MPI_Status* status);
int MPI_Cancel(MPI_Request* req);
int MPI_Request_free(MPI_Request* req);
int MPI_Get_count(const MPI_Status* status, MPI_Datatype type, int* count);
int MPI_Get_address(const void* location, MPI_Aint* address);
int MPI_Type_create_struct(int n, const int* lengths, const MPI_Aint* displs, const MPI_Datatype* types, MPI_Datatype* newtype);
int MPI_Type_commit(MPI_Datatype* type);
