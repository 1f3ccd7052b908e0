// Self-test of the local MPI subset (baseline/shims): two threads per rank exchange large and small messages around
// a ring with different tags (one side receiving from MPI_ANY_SOURCE), then every collective and an Irecv / Test
// polling loop are checked.  Exits 0 on success; any mismatch aborts.
#include "mpi.h"
#include <stdio.h>
#include <stdlib.h>
#include <thread>
#include <vector>
int main(int argc, char** argv) {
    int prov; MPI_Init_thread(&argc, &argv, MPI_THREAD_MULTIPLE, &prov);
    int r, n; MPI_Comm_rank(MPI_COMM_WORLD, &r); MPI_Comm_size(MPI_COMM_WORLD, &n);
    // ring with big messages, two threads with different tags
    std::vector<float> a(1 << 20, (float)r), b(1 << 20);
    auto ring = [&](int tag, std::vector<float>& s, std::vector<float>& d) {
        for (int it = 0; it < 5; ++it) {
            if (r % 2 == 0) { MPI_Send(s.data(), (int)s.size(), MPI_FLOAT, (r + 1) % n, tag, MPI_COMM_WORLD); MPI_Status st; MPI_Recv(d.data(), (int)d.size(), MPI_FLOAT, (r + n - 1) % n, tag, MPI_COMM_WORLD, &st); if (st.MPI_SOURCE != (r + n - 1) % n) abort(); }
            else { MPI_Status st; MPI_Recv(d.data(), (int)d.size(), MPI_FLOAT, MPI_ANY_SOURCE, tag, MPI_COMM_WORLD, &st); MPI_Send(s.data(), (int)s.size(), MPI_FLOAT, (r + 1) % n, tag, MPI_COMM_WORLD); }
            if (d[123] != (float)((r + n - 1) % n)) abort();
        }
    };
    std::vector<float> a2(1000, (float)r), b2(1000);
    std::thread t([&] { ring(7, a2, b2); });
    ring(3, a, b);
    t.join();
    double x = r + 1.0, s = 0; MPI_Allreduce(&x, &s, 1, MPI_DOUBLE, MPI_SUM, MPI_COMM_WORLD);
    if (s != n * (n + 1) / 2.0) abort();
    double y = r; MPI_Allreduce(MPI_IN_PLACE, &y, 1, MPI_DOUBLE, MPI_SUM, MPI_COMM_WORLD);
    if (y != n * (n - 1) / 2.0) abort();
    int mine = r * 10; std::vector<int> all(n); MPI_Allgather(&mine, 1, MPI_INT, all.data(), 1, MPI_INT, MPI_COMM_WORLD);
    for (int i = 0; i < n; ++i) if (all[i] != i * 10) abort();
    int v = r == 2 % n ? 99 : 0; MPI_Bcast(&v, 1, MPI_INT, 2 % n, MPI_COMM_WORLD); if (v != 99) abort();
    // Irecv + Test polling
    int got = -1; MPI_Request q; MPI_Irecv(&got, 1, MPI_INT, MPI_ANY_SOURCE, 11, MPI_COMM_WORLD, &q);
    MPI_Barrier(MPI_COMM_WORLD);
    int payload = 1000 + r; MPI_Send(&payload, 1, MPI_INT, (r + 1) % n, 11, MPI_COMM_WORLD);
    int flag = 0; MPI_Status st; while (!flag) MPI_Test(&q, &flag, &st);
    if (got != 1000 + (r + n - 1) % n) abort();
    MPI_Barrier(MPI_COMM_WORLD);
    if (r == 0) printf("mpi shim selftest ok on %d ranks\n", n);
    MPI_Finalize();
    return 0;
}
