// Forwards to the single shim header (same directory layout as the reference so its include paths resolve).
#pragma once
#include "../seblas.cuh"
