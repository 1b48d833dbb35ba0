// Handle types shared by the extern "C" translation units.
#pragma once

#include "host/graph.h"

struct nrs_node {
  nrs::NodeP p;
};
