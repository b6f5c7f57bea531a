// Same path as the reference header of this name; everything lives in ../seblas.cuh.
#pragma once
#include "../seblas.cuh"
