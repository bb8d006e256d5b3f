// Host-side rendezvous for one-process-per-rank runs: a TCP star through rank 0 for small
// all-gathers and barriers, and abstract-namespace unix sockets to pass file descriptors
// (the shareable handles of cuMem allocations) between the ranks of one host.
//
// Stands in for the TCP bootstrap the reference hands to its SHMEM library
// (utils/shmem_init.h:18-45: ip_port string, rank, world, timeouts).
#pragma once

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

namespace catccos {

class Bootstrap {
public:
    ~Bootstrap() { Close(); }

    // ip_port: "tcp://a.b.c.d:port" (the scheme is optional).  timeout_s bounds every blocking step.
    bool Init(int rank, int world, const char* ip_port, int timeout_s = 120)
    {
        rank_ = rank;
        world_ = world;
        timeout_s_ = timeout_s;
        std::string s = ip_port ? ip_port : "";
        size_t scheme = s.find("://");
        if (scheme != std::string::npos) {
            s = s.substr(scheme + 3);
        }
        size_t colon = s.rfind(':');
        if (colon == std::string::npos) {
            return Fail("rendezvous string needs ip:port");
        }
        ip_ = s.substr(0, colon);
        port_ = atoi(s.c_str() + colon + 1);
        if (port_ <= 0 || port_ > 65535) {
            return Fail("bad port");
        }
        if (world == 1) {
            return true;
        }
        return rank == 0 ? InitRoot() : InitLeaf();
    }

    // Every rank contributes `bytes`; recv gets world * bytes in rank order.
    bool AllGather(const void* send, void* recv, size_t bytes)
    {
        if (world_ == 1) {
            memcpy(recv, send, bytes);
            return true;
        }
        if (rank_ == 0) {
            std::vector<char> all(bytes * world_);
            memcpy(all.data(), send, bytes);
            for (int r = 1; r < world_; ++r) {
                if (!RecvAll(peers_[r], all.data() + bytes * r, bytes)) {
                    return Fail("allgather recv");
                }
            }
            for (int r = 1; r < world_; ++r) {
                if (!SendAll(peers_[r], all.data(), all.size())) {
                    return Fail("allgather send");
                }
            }
            memcpy(recv, all.data(), all.size());
            return true;
        }
        return (SendAll(root_, send, bytes) && RecvAll(root_, recv, bytes * world_)) || Fail("allgather leaf");
    }

    bool Barrier()
    {
        std::vector<int> v(world_);
        int mine = rank_;
        return AllGather(&mine, v.data(), sizeof(int));
    }

    // Every rank passes one file descriptor to every other rank.  fds_out[r] is a descriptor for
    // rank r's object valid in this process (fds_out[rank] = my_fd).
    bool ExchangeFds(int my_fd, std::vector<int>& fds_out)
    {
        fds_out.assign(world_, -1);
        fds_out[rank_] = my_fd;
        if (world_ == 1) {
            return true;
        }
        int seq = fd_seq_++;
        int lfd = socket(AF_UNIX, SOCK_STREAM, 0);
        if (lfd < 0) {
            return Fail("unix socket");
        }
        sockaddr_un addr;
        socklen_t alen = UnixName(rank_, seq, addr);
        if (bind(lfd, (sockaddr*)&addr, alen) != 0 || listen(lfd, world_ + 4) != 0) {
            close(lfd);
            return Fail("unix bind/listen");
        }
        bool ok = Barrier();  // every listener exists before anybody connects
        for (int r = 0; ok && r < world_; ++r) {
            if (r == rank_) {
                continue;
            }
            int c = socket(AF_UNIX, SOCK_STREAM, 0);
            sockaddr_un peer;
            socklen_t plen = UnixName(r, seq, peer);
            if (c < 0 || connect(c, (sockaddr*)&peer, plen) != 0) {
                ok = Fail("unix connect");
            } else {
                ok = SendFd(c, rank_, my_fd);
            }
            if (c >= 0) {
                close(c);
            }
        }
        for (int i = 0; ok && i < world_ - 1; ++i) {
            if (!WaitReadable(lfd)) {
                ok = Fail("unix accept timeout");
                break;
            }
            int c = accept(lfd, nullptr, nullptr);
            int from = -1, fd = -1;
            if (c < 0 || !RecvFd(c, from, fd) || from < 0 || from >= world_) {
                ok = Fail("unix recv fd");
            } else {
                fds_out[from] = fd;
            }
            if (c >= 0) {
                close(c);
            }
        }
        close(lfd);
        return ok && Barrier();
    }

    void Close()
    {
        for (int fd : peers_) {
            if (fd >= 0) {
                close(fd);
            }
        }
        peers_.clear();
        if (root_ >= 0) {
            close(root_);
            root_ = -1;
        }
    }

    const std::string& error() const { return err_; }

private:
    bool Fail(const char* what)
    {
        err_ = std::string(what) + ": " + strerror(errno);
        return false;
    }

    bool InitRoot()
    {
        int lfd = socket(AF_INET, SOCK_STREAM, 0);
        int one = 1;
        setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in a = {};
        a.sin_family = AF_INET;
        a.sin_port = htons((uint16_t)port_);
        a.sin_addr.s_addr = htonl(INADDR_ANY);
        if (bind(lfd, (sockaddr*)&a, sizeof(a)) != 0 || listen(lfd, world_ + 4) != 0) {
            close(lfd);
            return Fail("tcp bind/listen");
        }
        peers_.assign(world_, -1);
        for (int i = 1; i < world_; ++i) {
            if (!WaitReadable(lfd)) {
                close(lfd);
                return Fail("tcp accept timeout");
            }
            int c = accept(lfd, nullptr, nullptr);
            int r = -1;
            if (c < 0 || !RecvAll(c, &r, sizeof(r)) || r <= 0 || r >= world_ || peers_[r] >= 0) {
                close(lfd);
                return Fail("tcp accept");
            }
            setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            peers_[r] = c;
        }
        close(lfd);
        return true;
    }

    bool InitLeaf()
    {
        sockaddr_in a = {};
        a.sin_family = AF_INET;
        a.sin_port = htons((uint16_t)port_);
        if (inet_pton(AF_INET, ip_.c_str(), &a.sin_addr) != 1) {
            return Fail("bad ip");
        }
        time_t t0 = time(nullptr);
        while (true) {
            int c = socket(AF_INET, SOCK_STREAM, 0);
            if (connect(c, (sockaddr*)&a, sizeof(a)) == 0) {
                int one = 1;
                setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
                root_ = c;
                return SendAll(c, &rank_, sizeof(rank_)) || Fail("tcp hello");
            }
            close(c);
            if (time(nullptr) - t0 > timeout_s_) {
                return Fail("tcp connect timeout");
            }
            usleep(20000);
        }
    }

    socklen_t UnixName(int rank, int seq, sockaddr_un& addr) const
    {
        memset(&addr, 0, sizeof(addr));
        addr.sun_family = AF_UNIX;
        // abstract namespace: first byte of sun_path is 0, no file is created
        int n = snprintf(addr.sun_path + 1, sizeof(addr.sun_path) - 1, "catccos_b200.%d.%d.%d", port_, seq, rank);
        return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
    }

    bool WaitReadable(int fd) const
    {
        pollfd p = {fd, POLLIN, 0};
        return poll(&p, 1, timeout_s_ * 1000) == 1;
    }

    bool SendAll(int fd, const void* buf, size_t n)
    {
        const char* p = (const char*)buf;
        while (n > 0) {
            ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
            if (w <= 0) {
                if (w < 0 && errno == EINTR) {
                    continue;
                }
                return false;
            }
            p += w;
            n -= (size_t)w;
        }
        return true;
    }

    bool RecvAll(int fd, void* buf, size_t n)
    {
        char* p = (char*)buf;
        while (n > 0) {
            if (!WaitReadable(fd)) {
                return false;
            }
            ssize_t r = recv(fd, p, n, 0);
            if (r <= 0) {
                if (r < 0 && errno == EINTR) {
                    continue;
                }
                return false;
            }
            p += r;
            n -= (size_t)r;
        }
        return true;
    }

    bool SendFd(int sock, int from_rank, int fd)
    {
        msghdr msg = {};
        iovec iov = {&from_rank, sizeof(from_rank)};
        char ctrl[CMSG_SPACE(sizeof(int))] = {};
        msg.msg_iov = &iov;
        msg.msg_iovlen = 1;
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        cmsghdr* c = CMSG_FIRSTHDR(&msg);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int));
        memcpy(CMSG_DATA(c), &fd, sizeof(int));
        return sendmsg(sock, &msg, MSG_NOSIGNAL) == (ssize_t)sizeof(from_rank) || Fail("sendmsg");
    }

    bool RecvFd(int sock, int& from_rank, int& fd)
    {
        if (!WaitReadable(sock)) {
            return false;
        }
        msghdr msg = {};
        iovec iov = {&from_rank, sizeof(from_rank)};
        char ctrl[CMSG_SPACE(sizeof(int))] = {};
        msg.msg_iov = &iov;
        msg.msg_iovlen = 1;
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        if (recvmsg(sock, &msg, 0) != (ssize_t)sizeof(from_rank)) {
            return false;
        }
        cmsghdr* c = CMSG_FIRSTHDR(&msg);
        if (c == nullptr || c->cmsg_type != SCM_RIGHTS) {
            return false;
        }
        memcpy(&fd, CMSG_DATA(c), sizeof(int));
        return true;
    }

    int rank_ = 0, world_ = 1, port_ = 0, timeout_s_ = 120;
    int root_ = -1;
    int fd_seq_ = 0;
    std::string ip_, err_;
    std::vector<int> peers_;
};

}  // namespace catccos
