// Version of the API this library implements (mscclpp::version() adds the build tag of this implementation).
#pragma once

#define MSCCLPP_MAJOR 0
#define MSCCLPP_MINOR 9
#define MSCCLPP_PATCH 0
#define MSCCLPP_VERSION (MSCCLPP_MAJOR * 10000 + MSCCLPP_MINOR * 100 + MSCCLPP_PATCH)
#define MSCCLPP_GIT_COMMIT "b200.1"
