// Error convention of the front end, same two behaviours as the reference's include/Ctorch_Error.h:
// log(ERROR, ...) prints, counts and CONTINUES (:353-405); throwException prints and throws
// std::runtime_error (:510-515).  No banner, no start-up sleep.
#pragma once
#include <atomic>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "Ctools.h"

namespace ctorch {

class Ctorch_Stats {
public:
    static Ctorch_Stats& getInstance() {
        static Ctorch_Stats s;
        return s;
    }
    std::atomic<uint64_t> errors{0}, warns{0}, fatals{0};
    PrintLevel level = PrintLevel::MINIUM;
    bool quiet = false;  // suppress printing entirely (tests)
};

class Ctorch_Error {
public:
    static void setPrintLevel(PrintLevel l) { Ctorch_Stats::getInstance().level = l; }
    static void setQuiet(bool q) { Ctorch_Stats::getInstance().quiet = q; }
    static uint64_t errorCount() { return Ctorch_Stats::getInstance().errors.load(); }

    static void log(ErrorLevel level, ErrorPlatform platform, ErrorType type, const std::string& msg) {
        Ctorch_Stats& st = Ctorch_Stats::getInstance();
        if (level == ErrorLevel::ERROR) st.errors++;
        else if (level == ErrorLevel::WARN) st.warns++;
        else if (level == ErrorLevel::FATAL) st.fatals++;
        if (st.quiet) return;
        if (st.level == PrintLevel::MEDIUM && level == ErrorLevel::TRACE) return;
        if (st.level == PrintLevel::MINIUM && (level == ErrorLevel::DEBUG || level == ErrorLevel::TRACE)) return;
        static const char* names[] = {"TRACE", "INFO", "DEBUG", "WARN", "ERROR", "FATAL"};
        std::fprintf(stderr, "[%s] [PLATFORM:%d] [TYPE:%d] %s\n", names[static_cast<int>(level)], static_cast<int>(platform),
                     static_cast<int>(type), msg.c_str());
    }
    static void trace(ErrorPlatform platform, const std::string& msg) {
        if (Ctorch_Stats::getInstance().level == PrintLevel::FULL) log(ErrorLevel::TRACE, platform, ErrorType::UNKNOWN, msg);
    }
    [[noreturn]] static void throwException(ErrorPlatform platform, ErrorType type, const std::string& msg) {
        log(ErrorLevel::ERROR, platform, type, msg);
        throw std::runtime_error(msg);
    }
};

}  // namespace ctorch
