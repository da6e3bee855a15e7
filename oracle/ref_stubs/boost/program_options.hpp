// Stand-in: the reference test utilities include boost::program_options but do not use it.
#pragma once
