#pragma once
#include "ZZ.h"
