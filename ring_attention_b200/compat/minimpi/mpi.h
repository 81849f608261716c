/*
 * minimpi: the small part of MPI that the reference's drivers use, for one node, over a
 * shared-memory file. It exists so that the reference's MPI programs (apps/ring_attention_cli)
 * build and run unchanged on a machine without an MPI installation. One process per rank,
 * started by the `mpirun` launcher beside this header (it sets MINIMPI_RANK / MINIMPI_SIZE /
 * MINIMPI_SHM). Without those variables a program runs as a single rank.
 *
 * Implemented: Init, Finalize, Comm_rank, Comm_size, Comm_split_type (the world is one
 * shared-memory node), Comm_split (same colour everywhere only), Comm_free, Barrier, Bcast,
 * Reduce / Allreduce (MAX, MIN, SUM on int, float, double), Allgather, Wtime, Abort,
 * Error_string. Point-to-point calls are not provided: K/V travel over NCCL.
 */
#ifndef MINIMPI_MPI_H_
#define MINIMPI_MPI_H_

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Info;

#define MPI_COMM_WORLD 0
#define MPI_COMM_NULL (-1)
#define MPI_INFO_NULL 0
#define MPI_COMM_TYPE_SHARED 1
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_MAX_ERROR_STRING 256
#define MPI_IN_PLACE ((void*)1)

#define MPI_BYTE 1
#define MPI_CHAR 2
#define MPI_INT 3
#define MPI_UNSIGNED 4
#define MPI_FLOAT 5
#define MPI_DOUBLE 6
#define MPI_LONG 7
#define MPI_LONG_LONG 8

#define MPI_MAX 1
#define MPI_MIN 2
#define MPI_SUM 3

int MPI_Init(int* argc, char*** argv);
int MPI_Finalize(void);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_split_type(MPI_Comm comm, int split_type, int key, MPI_Info info, MPI_Comm* out);
int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* out);
int MPI_Comm_free(MPI_Comm* comm);
int MPI_Barrier(MPI_Comm comm);
int MPI_Bcast(void* buf, int count, MPI_Datatype type, int root, MPI_Comm comm);
int MPI_Reduce(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op, int root,
               MPI_Comm comm);
int MPI_Allreduce(const void* send, void* recv, int count, MPI_Datatype type, MPI_Op op,
                  MPI_Comm comm);
int MPI_Allgather(const void* send, int scount, MPI_Datatype stype, void* recv, int rcount,
                  MPI_Datatype rtype, MPI_Comm comm);
double MPI_Wtime(void);
int MPI_Abort(MPI_Comm comm, int code);
int MPI_Error_string(int code, char* str, int* len);

#ifdef __cplusplus
}
#endif
#endif
