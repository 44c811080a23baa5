#pragma once

#include "cell/copy/constants.hpp"
#include "cell/copy/global_to_register.hpp"
#include "cell/copy/global_to_shared.hpp"
#include "cell/copy/register.hpp"
#include "cell/copy/shared_to_register.hpp"
#include "cell/copy/tmem.hpp"
#include "cell/copy/warp.hpp"
