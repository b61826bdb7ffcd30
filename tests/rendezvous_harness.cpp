// Test harness for csrc/rank_rendezvous.h (host only): forks `ranks` processes that meet `points` times.
//   mode ok      : every rank arrives every time                     -> all exit 0
//   mode fail    : rank 1 raises the stop flag after 2 points, exits 7 -> the others leave with RV_STOPPED (exit 10 + 1)
//   mode vanish  : rank 1 exits after 2 points without a word; the parent raises the flag when it sees the exit
//   mode late    : rank 1 never arrives at point 3; the others give up after the time limit (RV_TIMEOUT or RV_STOPPED)
// Prints one line per rank: "rank r result <code> points <n> seconds <t>".
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "rank_rendezvous.h"

int main(int argc, char** argv) {
    const char* mode = argc > 1 ? argv[1] : "ok";
    const int ranks = argc > 2 ? atoi(argv[2]) : 4;
    const int points = argc > 3 ? atoi(argv[3]) : 100;
    const double limit = argc > 4 ? atof(argv[4]) : 5.0;
    b200::RendezvousPage* page = b200::rendezvous_create(ranks);
    if (!page) return 2;
    std::vector<pid_t> kids;
    for (int r = 0; r < ranks; ++r) {
        const pid_t pid = fork();
        if (pid == 0) {
            const double t0 = b200::rendezvous_now();
            int done = 0, res = b200::RV_OK;
            for (int p = 0; p < points; ++p) {
                if (r == 1 && p == 2) {
                    if (!strcmp(mode, "fail")) { b200::rendezvous_fail(page, r); _exit(7); }
                    if (!strcmp(mode, "vanish")) _exit(8);
                    if (!strcmp(mode, "late")) { sleep(3); _exit(9); }
                }
                res = b200::rendezvous_arrive(page, r, limit);
                if (res != b200::RV_OK) break;
                ++done;
            }
            printf("rank %d result %d points %d seconds %.3f\n", r, res, done, b200::rendezvous_now() - t0);
            fflush(stdout);
            _exit(res == b200::RV_OK ? 0 : 10 + res);
        }
        kids.push_back(pid);
    }
    int rc = 0;
    for (size_t i = 0; i < kids.size(); ++i) {
        int status = 0;
        const pid_t pid = wait(&status);
        const bool ok = pid > 0 && WIFEXITED(status) && WEXITSTATUS(status) == 0;
        if (!ok) {
            int which = -1;
            for (size_t r = 0; r < kids.size(); ++r)
                if (kids[r] == pid) which = static_cast<int>(r);
            b200::rendezvous_fail(page, which);  // what the training driver's parent does
            rc = 1;
        }
    }
    printf("failed_rank %d\n", page->failed_rank.load());
    b200::rendezvous_destroy(page);
    return rc;
}
