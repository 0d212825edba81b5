// Test infrastructure (oracle build only): see avx2.h in this folder.
#pragma once
#include "avx2.h"
