// Stand-in for <NTL/RR.h>; see ZZ.h beside this file.
#pragma once
#include "ZZ.h"
