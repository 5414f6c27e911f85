/* A stand-in for libnccl.so.2 whose communicator can never be initialised: the eight entry points the
 * fleet binds exist, ncclGetUniqueId works, and both init calls fail.  Test infrastructure: it lets the
 * "communicator not ready" path run on one GPU and without any faulting device code. */
#include <stddef.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void *ncclComm_t;
typedef void *cudaStream_t;

int ncclGetUniqueId(ncclUniqueId *id) { memset(id, 7, sizeof(*id)); return 0; }
int ncclCommInitRank(ncclComm_t *comm, int nranks, ncclUniqueId id, int rank) { (void)comm; (void)nranks; (void)id; (void)rank; return 3; }
int ncclCommInitAll(ncclComm_t *comm, int ndev, const int *devlist) { (void)comm; (void)ndev; (void)devlist; return 3; }
int ncclCommDestroy(ncclComm_t comm) { (void)comm; return 0; }
int ncclAllReduce(const void *s, void *r, size_t n, int t, int op, ncclComm_t c, cudaStream_t st) {
    (void)s; (void)r; (void)n; (void)t; (void)op; (void)c; (void)st; return 5;
}
int ncclGroupStart(void) { return 0; }
int ncclGroupEnd(void) { return 0; }
const char *ncclGetErrorString(int result) { return result == 0 ? "no error" : "communicator refused by the stand-in library"; }
