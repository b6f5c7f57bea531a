// Stand-in for the reference's seio/logging/LogUtils.cuh (which pulls in <windows.h>). The reference build
// recipe predefines that header's include guard and force-includes this file instead, so the reference's
// seblas sources compile untouched where they lie.
#pragma once
#include <chrono>
#include <cstdio>
#include <iostream>
#include <stdexcept>
#include <string>
using namespace std;
namespace seio {
enum LogSegments { LOG_SEG_SEIO = 0, LOG_SEG_SEANN = 1, LOG_SEG_SEBLAS = 2 };
inline void logInfo(LogSegments, const string& m) { fprintf(stderr, "[ref info] %s\n", m.c_str()); }
inline void logDebug(LogSegments, const string& m) { fprintf(stderr, "[ref debug] %s\n", m.c_str()); }
inline void logWarn(LogSegments, const string& m) { fprintf(stderr, "[ref warn] %s\n", m.c_str()); }
inline void logError(LogSegments, const string& m) { fprintf(stderr, "[ref error] %s\n", m.c_str()); }
inline void logFatal(LogSegments, const string& m) { fprintf(stderr, "[ref fatal] %s\n", m.c_str()); }
}  // namespace seio
