/* Stand-in for libnccl, for the watchdog tests only: a one-rank "communicator" whose all-reduce
 * keeps the stream busy from the HOST (a host function that sleeps; no GPU kernel spins) and
 * whose asynchronous error state can be made to report a failure.  FAKE_NCCL_MODE: 1 = the
 * collective stalls for 400 ms and the communicator reports an error, 2 = it only stalls. */
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef int (*launch_host_fn)(void* stream, void (*fn)(void*), void* data);

static int calls = 0;
static int mode(void) { const char* m = getenv("FAKE_NCCL_MODE"); return m ? atoi(m) : 0; }
static void sleeper(void* ms) { usleep((useconds_t)(long)ms * 1000); }

int ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(void** comm, int nranks, ncclUniqueId id, int rank) {
  (void)nranks; (void)id; (void)rank;
  *comm = malloc(16);
  return *comm ? 0 : 1;
}
int ncclAllReduce(const void* send, void* recv, size_t count, int dtype, int op, void* comm, void* stream) {
  (void)send; (void)recv; (void)count; (void)dtype; (void)op; (void)comm;
  ++calls;
  if (mode() == 0) return 0;                       /* the sum over one rank: nothing to do */
  void* cu = dlopen("libcuda.so.1", RTLD_NOW);
  launch_host_fn launch = cu ? (launch_host_fn)dlsym(cu, "cuLaunchHostFunc") : NULL;
  if (!launch) return 1;
  return launch(stream, sleeper, (void*)400L) ? 1 : 0;
}
int ncclCommGetAsyncError(void* comm, int* state) {
  (void)comm;
  *state = (mode() == 1 && calls > 0) ? 2 /* ncclSystemError */ : 0;
  return 0;
}
int ncclCommAbort(void* comm) { free(comm); return 0; }
int ncclCommDestroy(void* comm) { free(comm); return 0; }
const char* ncclGetErrorString(int code) { (void)code; return "stand-in library"; }
