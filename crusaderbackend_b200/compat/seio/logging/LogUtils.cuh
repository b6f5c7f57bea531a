// Portable stand-in for the reference's seio/logging/LogUtils.cuh (whose implementation drives the Win32 console):
// the same enums and function names, printing plain lines to stdout / stderr. Set CRUSADER_QUIET=1 to silence the
// info and debug levels.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <string>

namespace seio {

enum LogLevel { LOG_LEVEL_DEBUG = 0, LOG_LEVEL_INFO = 1, LOG_LEVEL_WARN = 2, LOG_LEVEL_ERROR = 3, LOG_LEVEL_FATAL = 4 };
enum LogSegments { LOG_SEG_SEIO = 0, LOG_SEG_SEANN = 1, LOG_SEG_SEBLAS = 2 };
enum LogColor {
    LOG_COLOR_RED, LOG_COLOR_LIGHT_RED, LOG_COLOR_GREEN, LOG_COLOR_LIGHT_GREEN, LOG_COLOR_YELLOW, LOG_COLOR_LIGHT_YELLOW,
    LOG_COLOR_BLUE, LOG_COLOR_LIGHT_BLUE, LOG_COLOR_AQUA, LOG_COLOR_LIGHT_AQUA, LOG_COLOR_PURPLE, LOG_COLOR_LIGHT_PURPLE,
    LOG_COLOR_WHITE, LOG_COLOR_BRIGHT_WHITE,
};

inline bool logQuiet() {
    static const bool q = std::getenv("CRUSADER_QUIET") != nullptr;
    return q;
}
inline void logLine(FILE* to, LogLevel level, LogSegments seg, const std::string& msg) {
    static const char* lv[] = {"DEBUG", "INFO", "WARN", "ERROR", "FATAL"};
    static const char* sg[] = {"seio", "seann", "seblas"};
    std::fprintf(to, "[%s|%s] %s\n", lv[level], sg[seg], msg.c_str());
}
inline void printLogHead(LogLevel level, LogSegments seg) { logLine(stdout, level, seg, ""); }
inline void logInfo(LogSegments seg, std::string msg) { if (!logQuiet()) logLine(stdout, LOG_LEVEL_INFO, seg, msg); }
inline void logInfo(LogSegments seg, const std::string& msg, LogColor) { logInfo(seg, msg); }
inline void logDebug(LogSegments seg, std::string msg) { if (!logQuiet()) logLine(stdout, LOG_LEVEL_DEBUG, seg, msg); }
inline void logDebug(LogSegments seg, const std::string& msg, LogColor) { logDebug(seg, msg); }
inline void logWarn(LogSegments seg, std::string msg) { logLine(stderr, LOG_LEVEL_WARN, seg, msg); }
inline void logError(LogSegments seg, std::string msg) { logLine(stderr, LOG_LEVEL_ERROR, seg, msg); }
inline void logFatal(LogSegments seg, std::string msg) { logLine(stderr, LOG_LEVEL_FATAL, seg, msg); }
inline void logProc(unsigned int proc, unsigned int finish) {
    if (!logQuiet()) std::printf("progress %u / %u\n", proc, finish);
}
inline void logTrainingProcess(unsigned int batchId, unsigned int epochId, unsigned int batches, unsigned int epochs,
                               float loss, float acc, float epochLoss, float epochAcc) {
    if (!logQuiet())
        std::printf("epoch %u/%u batch %u/%u loss %f acc %f (epoch loss %f acc %f)\n", epochId, epochs, batchId, batches, loss,
                    acc, epochLoss, epochAcc);
}

}  // namespace seio
