// see sycl.hpp beside this file
#pragma once
#include "sycl.hpp"
