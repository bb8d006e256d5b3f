// Host-only self test of the rendezvous layer (catccos_b200/csrc/bootstrap.hpp): forks `world`
// processes that meet over TCP on 127.0.0.1, all-gather a word, and pass one file descriptor each to
// every peer over abstract unix sockets (the path cuMem shareable handles take).  Each descriptor is
// a pipe whose payload names its owner, so a mix-up of ranks is caught.
//   usage: bootstrap_selftest <world> <port>      exit code 0 = pass
#include <sys/wait.h>

#include <cstdio>
#include <cstdlib>

#include "../../catccos_b200/csrc/bootstrap.hpp"

static int run_rank(int rank, int world, int port)
{
    catccos::Bootstrap b;
    char addr[64];
    snprintf(addr, sizeof(addr), "tcp://127.0.0.1:%d", port);
    if (!b.Init(rank, world, addr, 20)) {
        fprintf(stderr, "rank %d init: %s\n", rank, b.error().c_str());
        return 1;
    }
    std::vector<int> all(world, -1);
    int mine = rank * 7 + 1;
    if (!b.AllGather(&mine, all.data(), sizeof(int))) {
        return 2;
    }
    for (int r = 0; r < world; ++r) {
        if (all[r] != r * 7 + 1) {
            return 3;
        }
    }
    for (int round = 0; round < 2; ++round) {  // two exchanges: the socket names must not collide
        int pfd[2];
        if (pipe(pfd) != 0) {
            return 4;
        }
        int tag = rank * 100 + round;
        // one copy of the tag per reader (every peer reads once, and so does the owner below)
        for (int i = 0; i < world; ++i) {
            if (write(pfd[1], &tag, sizeof(tag)) != (ssize_t)sizeof(tag)) {
                return 5;
            }
        }
        std::vector<int> fds;
        if (!b.ExchangeFds(pfd[0], fds)) {
            fprintf(stderr, "rank %d exchange: %s\n", rank, b.error().c_str());
            return 6;
        }
        for (int r = 0; r < world; ++r) {
            int got = -1;
            if (read(fds[r], &got, sizeof(got)) != (ssize_t)sizeof(got) || got != r * 100 + round) {
                fprintf(stderr, "rank %d: descriptor of rank %d carries %d\n", rank, r, got);
                return 7;
            }
        }
        if (!b.Barrier()) {
            return 8;
        }
        for (int r = 0; r < world; ++r) {
            close(fds[r]);
        }
        close(pfd[1]);
    }
    return 0;
}

int main(int argc, char** argv)
{
    int world = argc > 1 ? atoi(argv[1]) : 2;
    int port = argc > 2 ? atoi(argv[2]) : 29917;
    std::vector<pid_t> kids;
    for (int r = 1; r < world; ++r) {
        pid_t p = fork();
        if (p == 0) {
            _exit(run_rank(r, world, port));
        }
        kids.push_back(p);
    }
    int rc = run_rank(0, world, port);
    for (pid_t p : kids) {
        int st = 0;
        waitpid(p, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
            rc = rc ? rc : 100 + (WIFEXITED(st) ? WEXITSTATUS(st) : 99);
        }
    }
    printf(rc == 0 ? "PASS\n" : "FAIL %d\n", rc);
    return rc;
}
