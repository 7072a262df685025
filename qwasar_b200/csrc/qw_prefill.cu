// placeholder until the tcgen05 kernel lands
#include "qw_kernels.h"
