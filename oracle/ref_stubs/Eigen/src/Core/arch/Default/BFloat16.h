#pragma once
#include <Eigen/Core>
