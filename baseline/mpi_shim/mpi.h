/* Single-node MPI subset over POSIX shared memory.
 *
 * Exists only so that the unmodified reference sources (C++ + MPI) can be built
 * and timed on a box that has no MPI installation.  It implements the calls
 * those sources use -- point-to-point with tags, the collectives, Cartesian
 * topologies, derived datatypes used for sends, and MPI-IO reads -- for ranks
 * that are processes of one machine.  Ranks are started by any launcher that
 * sets SP3MPI_RANK, SP3MPI_SIZE and SP3MPI_JOB in the environment.
 */
#ifndef SP3_MPI_SHIM_H
#define SP3_MPI_SHIM_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Request;
typedef int MPI_Info;
typedef int MPI_File;
typedef ptrdiff_t MPI_Aint;
typedef long long MPI_Offset;
typedef struct { int MPI_SOURCE, MPI_TAG, MPI_ERROR; } MPI_Status;

#define MPI_SUCCESS 0
#define MPI_COMM_NULL 0
#define MPI_COMM_WORLD 1
#define MPI_INFO_NULL 0
#define MPI_REQUEST_NULL 0

#define MPI_DATATYPE_NULL 0
#define MPI_CHAR 1
#define MPI_INT 2
#define MPI_UNSIGNED 3
#define MPI_UNSIGNED_LONG 4
#define MPI_DOUBLE 5
#define MPI_2INT 6
#define MPI_FLOAT 7
#define MPI_LONG_LONG 8
#define MPI_BYTE 9

#define MPI_SUM 1
#define MPI_MAX 2
#define MPI_MIN 3
#define MPI_MAXLOC 4

#define MPI_IN_PLACE ((void*)(intptr_t)-1)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)
#define MPI_WEIGHTS_EMPTY ((int*)0)
#define MPI_UNWEIGHTED ((int*)0)
#define MPI_MODE_RDONLY 1
#define MPI_SEEK_SET 0
#define MPI_SEEK_CUR 1
#define MPI_ANY_TAG (-1)
#define MPI_ANY_SOURCE (-2)

int MPI_Init(int* argc, char*** argv);
int MPI_Finalize(void);
int MPI_Abort(MPI_Comm comm, int code);
double MPI_Wtime(void);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_free(MPI_Comm* comm);
int MPI_Barrier(MPI_Comm comm);

int MPI_Send(const void* buf, int count, MPI_Datatype t, int dest, int tag, MPI_Comm comm);
int MPI_Recv(void* buf, int count, MPI_Datatype t, int src, int tag, MPI_Comm comm, MPI_Status* st);
int MPI_Irecv(void* buf, int count, MPI_Datatype t, int src, int tag, MPI_Comm comm, MPI_Request* rq);
int MPI_Wait(MPI_Request* rq, MPI_Status* st);
int MPI_Waitall(int n, MPI_Request* rq, MPI_Status* st);

int MPI_Bcast(void* buf, int count, MPI_Datatype t, int root, MPI_Comm comm);
int MPI_Ibcast(void* buf, int count, MPI_Datatype t, int root, MPI_Comm comm, MPI_Request* rq);
int MPI_Reduce(const void* s, void* r, int count, MPI_Datatype t, MPI_Op op, int root, MPI_Comm comm);
int MPI_Allreduce(const void* s, void* r, int count, MPI_Datatype t, MPI_Op op, MPI_Comm comm);
int MPI_Reduce_scatter(const void* s, void* r, const int* counts, MPI_Datatype t, MPI_Op op, MPI_Comm comm);
int MPI_Alltoall(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, MPI_Comm comm);
int MPI_Alltoallv(const void* s, const int* sc, const int* sd, MPI_Datatype st, void* r, const int* rc,
                  const int* rd, MPI_Datatype rt, MPI_Comm comm);
int MPI_Allgatherv(const void* s, int sc, MPI_Datatype st, void* r, const int* rc, const int* rd,
                   MPI_Datatype rt, MPI_Comm comm);
int MPI_Neighbor_alltoallv(const void* s, const int* sc, const int* sd, MPI_Datatype st, void* r,
                           const int* rc, const int* rd, MPI_Datatype rt, MPI_Comm comm);
int MPI_Dist_graph_create_adjacent(MPI_Comm comm, int indeg, const int* srcs, const int* sw, int outdeg,
                                   const int* dsts, const int* dw, MPI_Info info, int reorder, MPI_Comm* out);

int MPI_Dims_create(int nnodes, int ndims, int* dims);
int MPI_Cart_create(MPI_Comm comm, int ndims, const int* dims, const int* periods, int reorder, MPI_Comm* out);
int MPI_Cart_sub(MPI_Comm comm, const int* remain, MPI_Comm* out);
int MPI_Cart_get(MPI_Comm comm, int maxdims, int* dims, int* periods, int* coords);
int MPI_Cart_coords(MPI_Comm comm, int rank, int maxdims, int* coords);
int MPI_Cart_rank(MPI_Comm comm, const int* coords, int* rank);

int MPI_Type_create_struct(int n, const int* blens, const MPI_Aint* disps, const MPI_Datatype* types,
                           MPI_Datatype* out);
int MPI_Type_create_indexed_block(int n, int blen, const int* disps, MPI_Datatype old, MPI_Datatype* out);
int MPI_Type_indexed(int n, const int* blens, const int* disps, MPI_Datatype old, MPI_Datatype* out);
int MPI_Type_commit(MPI_Datatype* t);
int MPI_Type_free(MPI_Datatype* t);

int MPI_File_open(MPI_Comm comm, const char* name, int mode, MPI_Info info, MPI_File* fh);
int MPI_File_read(MPI_File fh, void* buf, int count, MPI_Datatype t, MPI_Status* st);
int MPI_File_seek(MPI_File fh, MPI_Offset off, int whence);
int MPI_File_close(MPI_File* fh);

#ifdef __cplusplus
}
#endif
#endif
