// Logging, CUDA error reporting and binary file helpers of the host operator surface.
// Mirrors the behaviour callers of the reference rely on (utils/utils.h:24-140): "[INFO]/[WARN]/[ERROR]"
// prefixes on stdout, an error-check macro that prints "<file>:<line> cudaError:<n>" to stderr and
// carries on, ReadFile that insists on an exact size match, ReadFileOrThrow, and WriteFile that
// takes an exclusive lock and writes at an offset.
#ifndef CATCCOS_B200_HOST_UTILS_H
#define CATCCOS_B200_HOST_UTILS_H

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/file.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>
#include <string>

#define INFO_LOG(fmt, args...) fprintf(stdout, "[INFO] " fmt "\n", ##args)
#define WARN_LOG(fmt, args...) fprintf(stdout, "[WARN] " fmt "\n", ##args)
#define ERROR_LOG(fmt, args...) fprintf(stdout, "[ERROR] " fmt "\n", ##args)

// The reference's ACL_CHECK logs and continues; so does this one.
#define CUDA_CHECK(status)                                                                       \
    do {                                                                                         \
        cudaError_t catccos_err_ = (status);                                                     \
        if (catccos_err_ != cudaSuccess) {                                                       \
            std::cerr << __FILE__ << ":" << __LINE__ << " cudaError:" << (int)catccos_err_ << std::endl; \
        }                                                                                        \
    } while (0)

// Status codes of the C ABI are reported the same way.
#define CATCCOS_CHECK(status)                                                                    \
    do {                                                                                         \
        int catccos_rc_ = (status);                                                              \
        if (catccos_rc_ != 0) {                                                                  \
            std::cerr << __FILE__ << ":" << __LINE__ << " cudaError:" << catccos_rc_ << " (catccos_b200)" << std::endl; \
        }                                                                                        \
    } while (0)

inline bool ReadFile(const std::string& filePath, void* buffer, size_t bufferSize)
{
    struct stat info;
    if (stat(filePath.c_str(), &info) != 0) {
        ERROR_LOG("Failed to get file");
        return false;
    }
    if (!S_ISREG(info.st_mode)) {
        ERROR_LOG("%s is not a file, please enter a file.", filePath.c_str());
        return false;
    }
    if (info.st_size == 0) {
        ERROR_LOG("File size is 0");
        return false;
    }
    if (static_cast<size_t>(info.st_size) != bufferSize) {
        ERROR_LOG("File size does not match buffer size.");
        return false;
    }
    std::ifstream in(filePath, std::ios::binary);
    if (!in) {
        ERROR_LOG("Open file failed. path = %s.", filePath.c_str());
        return false;
    }
    in.read(static_cast<char*>(buffer), static_cast<std::streamsize>(bufferSize));
    if (static_cast<size_t>(in.gcount()) != bufferSize) {
        ERROR_LOG("Failed to read the complete file.");
        return false;
    }
    return true;
}

inline void ReadFileOrThrow(const std::string& filePath, void* buffer, size_t bufferSize)
{
    if (!ReadFile(filePath, buffer, bufferSize)) {
        throw std::runtime_error("Failed to read file: " + filePath);
    }
}

inline bool WriteFile(const std::string& filePath, const void* buffer, size_t size, size_t offset = 0)
{
    if (buffer == nullptr) {
        ERROR_LOG("Write file failed. Buffer is nullptr.");
        return false;
    }
    const int fd = open(filePath.c_str(), O_RDWR | O_CREAT, 0666);
    if (fd < 0) {
        ERROR_LOG("Open file failed. path = %s", filePath.c_str());
        return false;
    }
    bool ok = false;
    if (flock(fd, LOCK_EX) != 0) {
        std::cerr << "Failed to acquire lock: " << strerror(errno) << std::endl;
    } else {
        const ssize_t n = pwrite(fd, buffer, size, static_cast<off_t>(offset));
        if (n == static_cast<ssize_t>(size)) {
            ok = true;
        } else if (n < 0) {
            std::cerr << "Failed to write to file: " << strerror(errno) << std::endl;
        } else {
            std::cerr << "Incomplete file write: " << n << " of " << size << " bytes" << std::endl;
        }
        flock(fd, LOCK_UN);
    }
    close(fd);
    return ok;
}

#endif  // CATCCOS_B200_HOST_UTILS_H
