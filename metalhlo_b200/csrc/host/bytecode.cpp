// MLIR bytecode -> StableHLO text through a helper process.
//
// JAX hands a PJRT plugin its programs as MLIR bytecode (magic "ML\xEFR", a VHLO portable artifact). This backend parses
// text, and no MLIR bytecode reader is linked; like the reference (Sources/PJRTMetalHLO/PJRTExecutable.swift:23-239) it asks
// the Python interpreter that hosts JAX to deserialize the artifact with jaxlib and print it: the interpreter named by
// METALHLO_PYTHON (the jax_plugins.metalhlo package sets it to sys.executable), running the helper script named by
// METALHLO_BYTECODE_HELPER (default: jax_plugins/metalhlo/bytecode_to_text.py beside this library's package). The
// bytecode goes to the helper's stdin, the text comes back on its stdout; both pipes are serviced at the same time so
// that neither side can block the other, and the helper is given METALHLO_HELPER_TIMEOUT_S seconds (default 120) before
// the child this call started is killed.
#include <dlfcn.h>
#include <fcntl.h>
#include <poll.h>
#include <signal.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>

#include "compiler.h"

namespace mhlo {

bool is_mlir_bytecode(const char* data, size_t size) {
    return size >= 4 && static_cast<unsigned char>(data[0]) == 0x4D && static_cast<unsigned char>(data[1]) == 0x4C &&
           static_cast<unsigned char>(data[2]) == 0xEF && static_cast<unsigned char>(data[3]) == 0x52;
}

namespace {

std::string default_helper_path() {
    Dl_info info;
    if (dladdr(reinterpret_cast<const void*>(&is_mlir_bytecode), &info) == 0 || !info.dli_fname) return "";
    std::string lib = info.dli_fname;  // .../metalhlo_b200/lib/libCMetalHLO.so
    const size_t slash = lib.rfind('/');
    const std::string dir = slash == std::string::npos ? "." : lib.substr(0, slash);
    return dir + "/../python/jax_plugins/metalhlo/bytecode_to_text.py";
}

void set_nonblocking(int fd) {
    const int flags = fcntl(fd, F_GETFL, 0);
    if (flags >= 0) fcntl(fd, F_SETFL, flags | O_NONBLOCK);
}

}  // namespace

bool bytecode_to_text(const char* bytecode, size_t size, std::string* text, std::string* why) {
    const char* py = std::getenv("METALHLO_PYTHON");
    const std::string python = py && *py ? py : "python3";
    const char* hp = std::getenv("METALHLO_BYTECODE_HELPER");
    const std::string helper = hp && *hp ? hp : default_helper_path();
    if (helper.empty() || access(helper.c_str(), R_OK) != 0) {
        *why = "Bytecode conversion failed: helper script '" + helper + "' not found (set METALHLO_BYTECODE_HELPER)";
        return false;
    }
    double timeout_s = 120.0;
    if (const char* t = std::getenv("METALHLO_HELPER_TIMEOUT_S")) {
        const double v = std::atof(t);
        if (v > 0) timeout_s = v;
    }
    int in_pipe[2], out_pipe[2], err_pipe[2], exec_pipe[2];
    if (pipe(in_pipe) != 0 || pipe(out_pipe) != 0 || pipe(err_pipe) != 0 || pipe(exec_pipe) != 0) {
        *why = std::string("Bytecode conversion failed: pipe: ") + std::strerror(errno);
        return false;
    }
    fcntl(exec_pipe[1], F_SETFD, FD_CLOEXEC);  // closes on a successful exec; carries errno otherwise
    const pid_t pid = fork();
    if (pid < 0) {
        *why = std::string("Bytecode conversion failed: fork: ") + std::strerror(errno);
        for (int fd : {in_pipe[0], in_pipe[1], out_pipe[0], out_pipe[1], err_pipe[0], err_pipe[1], exec_pipe[0], exec_pipe[1]}) close(fd);
        return false;
    }
    if (pid == 0) {
        dup2(in_pipe[0], 0);
        dup2(out_pipe[1], 1);
        dup2(err_pipe[1], 2);
        for (int fd : {in_pipe[0], in_pipe[1], out_pipe[0], out_pipe[1], err_pipe[0], err_pipe[1], exec_pipe[0]}) close(fd);
        execlp(python.c_str(), python.c_str(), helper.c_str(), static_cast<char*>(nullptr));
        const int e = errno;
        if (write(exec_pipe[1], &e, sizeof e) < 0) {}
        _exit(127);
    }
    close(in_pipe[0]);
    close(out_pipe[1]);
    close(err_pipe[1]);
    close(exec_pipe[1]);
    int exec_errno = 0;
    const ssize_t got = read(exec_pipe[0], &exec_errno, sizeof exec_errno);
    close(exec_pipe[0]);
    if (got == static_cast<ssize_t>(sizeof exec_errno)) {
        close(in_pipe[1]);
        close(out_pipe[0]);
        close(err_pipe[0]);
        int status = 0;
        waitpid(pid, &status, 0);
        *why = "Bytecode conversion failed: Failed to launch Python '" + python + "': " + std::strerror(exec_errno);
        return false;
    }
    set_nonblocking(in_pipe[1]);
    set_nonblocking(out_pipe[0]);
    set_nonblocking(err_pipe[0]);
    const struct sigaction ignore = [] { struct sigaction a; std::memset(&a, 0, sizeof a); a.sa_handler = SIG_IGN; return a; }();
    struct sigaction old_pipe;
    sigaction(SIGPIPE, &ignore, &old_pipe);  // a helper that exits early must not kill the host with SIGPIPE
    std::string out, err;
    size_t written = 0;
    int in_fd = in_pipe[1], out_fd = out_pipe[0], err_fd = err_pipe[0];
    if (size == 0) { close(in_fd); in_fd = -1; }
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
    bool timed_out = false;
    char buf[65536];
    while (out_fd >= 0 || err_fd >= 0) {
        struct pollfd fds[3];
        int n = 0, in_slot = -1, out_slot = -1, err_slot = -1;
        if (in_fd >= 0) { fds[n] = {in_fd, POLLOUT, 0}; in_slot = n++; }
        if (out_fd >= 0) { fds[n] = {out_fd, POLLIN, 0}; out_slot = n++; }
        if (err_fd >= 0) { fds[n] = {err_fd, POLLIN, 0}; err_slot = n++; }
        const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now()).count();
        if (left <= 0) { timed_out = true; break; }
        const int ready = poll(fds, static_cast<nfds_t>(n), static_cast<int>(left > 1000 ? 1000 : left));
        if (ready < 0 && errno != EINTR) break;
        if (ready <= 0) continue;
        if (in_slot >= 0 && (fds[in_slot].revents & (POLLOUT | POLLERR | POLLHUP))) {
            const ssize_t w = write(in_fd, bytecode + written, size - written);
            if (w > 0) written += static_cast<size_t>(w);
            if (written == size || (w < 0 && errno != EAGAIN && errno != EINTR)) { close(in_fd); in_fd = -1; }
        }
        auto drain = [&](int* fd, int slot, std::string* dst) {
            if (slot < 0 || !(fds[slot].revents & (POLLIN | POLLHUP | POLLERR))) return;
            const ssize_t r = read(*fd, buf, sizeof buf);
            if (r > 0) dst->append(buf, static_cast<size_t>(r));
            else if (r == 0 || (errno != EAGAIN && errno != EINTR)) { close(*fd); *fd = -1; }
        };
        drain(&out_fd, out_slot, &out);
        drain(&err_fd, err_slot, &err);
    }
    for (int fd : {in_fd, out_fd, err_fd})
        if (fd >= 0) close(fd);
    sigaction(SIGPIPE, &old_pipe, nullptr);
    int status = 0;
    if (timed_out) {
        kill(pid, SIGKILL);  // the exact child this call started
        waitpid(pid, &status, 0);
        *why = "Bytecode conversion failed: the helper did not finish within " + std::to_string(static_cast<int>(timeout_s)) + " s";
        return false;
    }
    waitpid(pid, &status, 0);
    const int code = WIFEXITED(status) ? WEXITSTATUS(status) : 128 + (WIFSIGNALED(status) ? WTERMSIG(status) : 0);
    if (code != 0) {
        if (err.size() > 2000) err = err.substr(err.size() - 2000);
        *why = "Bytecode conversion failed: Python conversion failed (exit " + std::to_string(code) + "): " + (err.empty() ? "no message" : err);
        return false;
    }
    if (out.empty()) {
        *why = "Bytecode conversion failed: Python conversion produced empty output";
        return false;
    }
    *text = std::move(out);
    return true;
}

}  // namespace mhlo
