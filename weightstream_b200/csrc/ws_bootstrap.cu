// Bootstrap without a host framework: the ranks of a group trade their 128-byte IPC handles over TCP.
// Stands in for what the reference's control plane does for its ring (one TCP connection per rank to
// a rendezvous address, crates/weightstream-transport/src/ctrl.rs:12-29; group bring-up in
// crates/weightstream-gpu/src/tp4.rs:191-312).  Plain POSIX sockets, blocking with poll() deadlines.
//
// Protocol (rank 0 listens, ranks 1..world-1 connect, retrying until the deadline):
//   rank r -> rank 0 : {magic, rank, world, len} (4 x u32, little endian) then `len` bytes
//   rank 0 -> rank r : status (i32), then, if it is WS_OK, world * len bytes in rank order
//                      (after every rank has reported, or when rank 0 gives up)
// A rank that reports a wrong world or length, a rank number out of range or one that was already
// taken ends the rendezvous with WS_ERR_INVALID; a rank that never shows up with WS_ERR_TIMEOUT; rank 0
// tells the ranks that did connect which of the two it was.
#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <time.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "../../include/ws_tp.h"

namespace {

constexpr uint32_t kMagic = 0x57535450u;  // "WSTP"

int64_t now_ms() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

// Moves exactly `len` bytes or fails: 0 ok, -1 error / peer closed, -2 deadline passed.
int xfer(int fd, void *buf, size_t len, bool sending, int64_t deadline) {
    char *p = static_cast<char *>(buf);
    while (len > 0) {
        const int64_t left = deadline - now_ms();
        if (left <= 0) return -2;
        pollfd pf{fd, (short)(sending ? POLLOUT : POLLIN), 0};
        const int pr = poll(&pf, 1, (int)(left > 1000 ? 1000 : left));
        if (pr < 0 && errno != EINTR) return -1;
        if (pr <= 0) continue;
        const ssize_t n = sending ? send(fd, p, len, MSG_NOSIGNAL) : recv(fd, p, len, 0);
        if (n == 0 && !sending) return -1;
        if (n < 0) {
            if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
            return -1;
        }
        p += n;
        len -= (size_t)n;
    }
    return 0;
}

bool resolve(const char *host, int port, sockaddr_in *out) {
    memset(out, 0, sizeof *out);
    out->sin_family = AF_INET;
    out->sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host, &out->sin_addr) == 1) return true;
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(host, nullptr, &hints, &res) != 0 || !res) return false;
    out->sin_addr = reinterpret_cast<sockaddr_in *>(res->ai_addr)->sin_addr;
    freeaddrinfo(res);
    return true;
}

ws_status_t serve(int world, const sockaddr_in &addr, const void *in, void *out, uint32_t len, int64_t deadline) {
    const int ls = socket(AF_INET, SOCK_STREAM, 0);
    if (ls < 0) return WS_ERR_CUDA;
    int one = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    if (bind(ls, reinterpret_cast<const sockaddr *>(&addr), sizeof addr) != 0 || listen(ls, world) != 0) {
        close(ls);
        return WS_ERR_INVALID;
    }
    std::vector<int> fds(world, -1);
    char *all = static_cast<char *>(out);
    memcpy(all, in, len);
    ws_status_t st = WS_OK;
    for (int got = 1; got < world && st == WS_OK;) {
        const int64_t left = deadline - now_ms();
        if (left <= 0) { st = WS_ERR_TIMEOUT; break; }
        pollfd pf{ls, POLLIN, 0};
        const int pr = poll(&pf, 1, (int)(left > 1000 ? 1000 : left));
        if (pr < 0 && errno != EINTR) { st = WS_ERR_CUDA; break; }
        if (pr <= 0) continue;
        const int fd = accept(ls, nullptr, nullptr);
        if (fd < 0) continue;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
        uint32_t hdr[4];
        const int xr = xfer(fd, hdr, sizeof hdr, false, deadline);
        if (xr != 0) { close(fd); st = xr == -2 ? WS_ERR_TIMEOUT : WS_ERR_INVALID; break; }
        if (hdr[0] != kMagic || hdr[2] != (uint32_t)world || hdr[3] != len || hdr[1] == 0 || hdr[1] >= (uint32_t)world ||
            fds[hdr[1]] >= 0) {
            close(fd);
            st = WS_ERR_INVALID;  // a stranger, a different group, or a rank number given twice
            break;
        }
        if (xfer(fd, all + (size_t)hdr[1] * len, len, false, deadline) != 0) { close(fd); st = WS_ERR_TIMEOUT; break; }
        fds[hdr[1]] = fd;
        ++got;
    }
    const ws_status_t verdict = st;
    for (int r = 1; r < world; ++r) {
        if (fds[r] < 0) continue;
        int32_t word = (int32_t)verdict;
        const int64_t dl = verdict == WS_OK ? deadline : now_ms() + 200;  // the bad news may go out after the deadline
        if (xfer(fds[r], &word, sizeof word, true, dl) != 0) {
            if (st == WS_OK) st = WS_ERR_TIMEOUT;
        } else if (verdict == WS_OK && xfer(fds[r], all, (size_t)world * len, true, deadline) != 0) {
            st = WS_ERR_TIMEOUT;
        }
        close(fds[r]);
    }
    close(ls);
    return st;
}

ws_status_t join(int rank, int world, const sockaddr_in &addr, const void *in, void *out, uint32_t len, int64_t deadline) {
    for (;;) {  // the listener may not be up yet: retry until the deadline
        if (now_ms() >= deadline) return WS_ERR_TIMEOUT;
        const int fd = socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) return WS_ERR_CUDA;
        if (connect(fd, reinterpret_cast<const sockaddr *>(&addr), sizeof addr) != 0) {
            close(fd);
            timespec nap{0, 20 * 1000 * 1000};
            nanosleep(&nap, nullptr);
            continue;
        }
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
        uint32_t hdr[4] = {kMagic, (uint32_t)rank, (uint32_t)world, len};
        int xr = xfer(fd, hdr, sizeof hdr, true, deadline);
        if (xr == 0) xr = xfer(fd, const_cast<void *>(in), len, true, deadline);
        int32_t verdict = WS_OK;
        if (xr == 0) xr = xfer(fd, &verdict, sizeof verdict, false, deadline + 500);  // rank 0 reports a little after its own deadline
        if (xr == 0 && verdict == WS_OK) xr = xfer(fd, out, (size_t)world * len, false, deadline + 500);
        close(fd);
        if (xr == 0) return (ws_status_t)verdict;
        return xr == -2 ? WS_ERR_TIMEOUT : WS_ERR_INVALID;  // rank 0 turned this rank away at once, or went away itself
    }
}

}  // namespace

extern "C" {

ws_status_t ws_tcp_allgather(int32_t rank, int32_t world, const char *host, int32_t port, const void *in, void *out,
                             int32_t len, int32_t timeout_ms) {
    if (!host || !in || !out || world < 1 || world > WS_MAX_WORLD || rank < 0 || rank >= world || len < 1 || port < 1 ||
        port > 65535 || timeout_ms < 1)
        return WS_ERR_INVALID;
    if (world == 1) {
        memcpy(out, in, (size_t)len);
        return WS_OK;
    }
    sockaddr_in addr;
    if (!resolve(host, port, &addr)) return WS_ERR_INVALID;
    const int64_t deadline = now_ms() + timeout_ms;
    return rank == 0 ? serve(world, addr, in, out, (uint32_t)len, deadline) : join(rank, world, addr, in, out, (uint32_t)len, deadline);
}

ws_status_t ws_tp_connect_tcp(ws_tp_t *tp, int32_t rank, int32_t world, const char *host, int32_t port, int32_t timeout_ms) {
    if (!tp) return WS_ERR_INVALID;
    ws_ipc_handle_t mine;
    ws_status_t s = ws_tp_export_handle(tp, &mine);
    if (s != WS_OK) return s;
    std::vector<ws_ipc_handle_t> all((size_t)(world > 0 ? world : 1));
    s = ws_tcp_allgather(rank, world, host, port, &mine, all.data(), (int32_t)sizeof mine, timeout_ms);
    if (s != WS_OK) return s;
    return ws_tp_connect_ipc(tp, all.data(), world);  // checks world, rank order and layout of every handle
}

}  // extern "C"
